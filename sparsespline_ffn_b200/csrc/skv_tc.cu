// Entry points of the tcgen05 kernel family as seen by the C ABI.
#include "skv_tc_common.cuh"

namespace skv {
namespace tc {
bool fwd_eligible(const skv_problem& p);
bool bwd_eligible(const skv_problem& p);
size_t fwd_scratch_bytes(const skv_problem& p);
size_t bwd_scratch_bytes(const skv_problem& p);
int forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
            void* delta_out, int64_t ds, void* scratch, size_t scratch_bytes);
int backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
             const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast, void* scratch,
             size_t scratch_bytes);
}  // namespace tc

bool tc_eligible(const skv_problem& p) { return tc::fwd_eligible(p) && tc::bwd_eligible(p); }

size_t tc_scratch_bytes(const skv_problem& p, int op) {
  return op == SKV_OP_FORWARD ? tc::fwd_scratch_bytes(p) : tc::bwd_scratch_bytes(p);
}

int tc_forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
               void* delta_out, int64_t ds, void* scratch, size_t scratch_bytes) {
  return tc::forward(c, z, zs, C, act_out, as, delta_out, ds, scratch, scratch_bytes);
}

int tc_backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
                const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast,
                void* scratch, size_t scratch_bytes) {
  return tc::backward(c, z, zs, C, g_act, gas, g_delta, gds, dz, dzs, dC, dC_cast, scratch, scratch_bytes);
}

}  // namespace skv
