#include "skv_common.cuh"
namespace skv {
bool tc_eligible(const skv_problem&) { return false; }
size_t tc_scratch_bytes(const skv_problem&, int) { return 0; }
int tc_forward(const LaunchCtx&, const void*, int64_t, const void*, void*, int64_t, void*, int64_t, void*, size_t) { return SKV_ERR_UNSUPPORTED; }
int tc_backward(const LaunchCtx&, const void*, int64_t, const void*, const void*, int64_t, const void*, int64_t, void*, int64_t, float*, void*, void*, size_t) { return SKV_ERR_UNSUPPORTED; }
}
