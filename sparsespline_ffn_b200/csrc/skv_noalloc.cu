// Forward entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run the operator:
// inference servers with a fixed device-memory budget, plugin sandboxes that forbid allocation
// after start-up, and real-time loops where an allocation's latency and implicit synchronisation
// are not acceptable.  The regular forward asks such a caller for a
// scratch buffer it has no way to obtain.  This variant brings its own: a fixed array in the
// library's device image.
#include <mutex>

#include "skv_common.cuh"

// The scratch of the forward kernels (f16 operand image of the code table followed by the
// float32 partial residuals of the key splits) lives here.  Every GPU that loads the library
// holds these 16 MiB until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SKV_NOALLOC_SCRATCH_BYTES];

namespace {
std::mutex g_mu;
void* g_scratch_addr[64];   // device address of g_noalloc_scratch, per device ordinal

// In host code `g_noalloc_scratch` is only a handle of the symbol, not a device address, so the
// address a kernel can use is looked up once per device, with that device current.
int scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return SKV_ERR_DEVICE; }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) { cudaGetLastError(); return SKV_ERR_DEVICE; }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SKV_OK;
}
}  // namespace

extern "C" int skv_feature_forward_noalloc(const skv_problem* p, const void* z, int64_t z_stride, const void* C,
                                           void* act_out, int64_t act_stride, void* delta_out,
                                           int64_t delta_stride, int32_t* status, void* stream) {
  if (!p) return SKV_ERR_NULL;
  const int impl = skv_resolve_impl(p);
  if (impl < 0) return impl;
  const size_t need = skv_scratch_bytes(p, SKV_OP_FORWARD);
  if (need > (size_t)SKV_NOALLOC_SCRATCH_BYTES) return SKV_ERR_NOALLOC_LIMIT;
  void* scratch = nullptr;
  if (int e = scratch_address(&scratch)) return e;
  // Nothing in the array has to start at zero: the forward writes the whole operand image and
  // every partial-residual row it later reads before reading them, so leftovers of the previous
  // call are never observed.
  return skv_feature_forward(p, z, z_stride, C, act_out, act_stride, delta_out, delta_stride, scratch,
                             (size_t)SKV_NOALLOC_SCRATCH_BYTES, status, stream);
}
