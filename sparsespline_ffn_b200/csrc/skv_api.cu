// C ABI of the library (declared in include/splinekv_b200.h): argument validation, kernel-family
// choice, no allocation, no synchronisation.
#include <atomic>
#include <cstring>

#include "skv_common.cuh"

using namespace skv;

namespace skv {
static std::atomic<uint64_t> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// Debug / test settings (skv_debug_set), read by the launch code of the tensor-core kernels.
static std::atomic<long long> g_wait_cycles{4000000000LL};
static std::atomic<int> g_skip_copy{0};
static std::atomic<int> g_fused_bwd{0};
namespace tc {
long long wait_cycle_limit() { return g_wait_cycles.load(std::memory_order_relaxed); }
int debug_skip_copy() { return g_skip_copy.load(std::memory_order_relaxed); }
int fused_backward_roles() { return g_fused_bwd.load(std::memory_order_relaxed); }
}  // namespace tc
}  // namespace skv

namespace skv {
namespace tc {
bool readout_eligible(const skv_problem& p, int64_t D);
size_t readout_image_bytes(const skv_problem& p, int64_t D);
int64_t readout_delta_pitch(const skv_problem& p);
int readout(const LaunchCtx& c, const void* z, int64_t zs, const void* delta, const void* W, int64_t ws, int64_t D,
            void* y, int64_t ys, void* wimg);
}  // namespace tc
}  // namespace skv

namespace {

size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }

int validate(const skv_problem* p) {
  if (!p) return SKV_ERR_NULL;
  if (p->N < 0 || p->h < 1 || p->L < (p->spline_order == 1 ? 3 : 4) || p->r < 1) return SKV_ERR_SHAPE;
  if (p->N > (int64_t)1 << 40 || p->h > (1 << 24) || p->L > 4096) return SKV_ERR_SHAPE;
  if (p->dtype != SKV_BF16 && p->dtype != SKV_F32) return SKV_ERR_UNSUPPORTED;
  if (p->activation != SKV_ACT_RELU_SQ && p->activation != SKV_ACT_IDENTITY && p->activation != SKV_ACT_GELU)
    return SKV_ERR_UNSUPPORTED;
  if (p->impl != SKV_IMPL_AUTO && p->impl != SKV_IMPL_SIMT && p->impl != SKV_IMPL_TCGEN05)
    return SKV_ERR_UNSUPPORTED;
  if (p->r > 256) return SKV_ERR_UNSUPPORTED;
  if (p->spline_order != 0 && p->spline_order != 1 && p->spline_order != 2) return SKV_ERR_UNSUPPORTED;
  return SKV_OK;
}

int resolve(const skv_problem& p) {
  if (p.impl == SKV_IMPL_SIMT) return SKV_IMPL_SIMT;
  const bool ok = p.spline_order != 1 && tc_eligible(p);      // the linear spline runs on the CUDA-core kernels
  if (p.impl == SKV_IMPL_TCGEN05) return ok ? (int)SKV_IMPL_TCGEN05 : (int)SKV_ERR_UNSUPPORTED;
  return ok ? (int)SKV_IMPL_TCGEN05 : (int)SKV_IMPL_SIMT;
}

// Compute capability and SM count of the current device, cached per device ordinal.
struct DevInfo { int known, major, sms; };
DevInfo g_dev[64];

int device_info(int* sms) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return SKV_ERR_DEVICE; }
  DevInfo& d = g_dev[dev];
  if (!d.known) {
    int major = 0, n = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return SKV_ERR_DEVICE;
    }
    d.major = major;
    d.sms = n;
    d.known = 1;
  }
  if (d.major != 10) return SKV_ERR_DEVICE;
  if (sms) *sms = d.sms;
  return SKV_OK;
}

int make_ctx(const skv_problem* p, void* stream, int32_t* status, LaunchCtx* c) {
  if (int e = validate(p)) return e;
  int sms = 0;
  if (int e = device_info(&sms)) return e;
  c->p = *p;
  const int order = p->spline_order == 1 ? 1 : 2;
  c->G = p->L - order;
  c->g.lo = p->grid_lo;
  c->g.scale = p->scale;
  c->g.Gf = (float)(p->L - order);
  c->g.Gm1f = (float)(p->L - order - 1);
  c->g.order = order;
  c->stream = (cudaStream_t)stream;
  c->status = status;
  c->num_sms = sms;
  return SKV_OK;
}

bool aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

}  // namespace

extern "C" {

int skv_abi_version(void) { return SKV_ABI_VERSION; }

uint64_t skv_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

const char* skv_error_string(int code) {
  switch (code) {
    case SKV_OK: return "ok";
    case SKV_ERR_NULL: return "a required pointer is NULL";
    case SKV_ERR_SHAPE: return "bad shape: need N >= 0, h >= 1, L = G + spline_order with G >= 2, r >= 1";
    case SKV_ERR_UNSUPPORTED: return "unsupported dtype, activation, impl or r > 256 for this shape";
    case SKV_ERR_ALIGN: return "pointer or stride alignment required by the kernel is not met";
    case SKV_ERR_SCRATCH: return "scratch buffer missing or smaller than skv_scratch_bytes()";
    case SKV_ERR_DEVICE: return "current CUDA device is not compute capability 10.x (B200, sm_100a)";
    case SKV_ERR_LAUNCH: return "CUDA kernel launch failed";
    case SKV_ERR_NOALLOC_LIMIT:
      return "problem needs more scratch than the built-in SKV_NOALLOC_SCRATCH_BYTES array; use "
             "skv_feature_forward with caller-owned scratch";
    default: return "unknown error code";
  }
}

int skv_device_ok(void) { return device_info(nullptr); }

int skv_debug_set(int what, int64_t value) {
  switch (what) {
    case SKV_DEBUG_WAIT_CYCLES:
      if (value < 1000) return SKV_ERR_UNSUPPORTED;
      skv::g_wait_cycles.store((long long)value, std::memory_order_relaxed);
      return SKV_OK;
    case SKV_DEBUG_SKIP_FIRST_COPY:
      if (value < 0 || value > 2) return SKV_ERR_UNSUPPORTED;
      skv::g_skip_copy.store((int)value, std::memory_order_relaxed);
      return SKV_OK;
    case SKV_DEBUG_FUSED_BACKWARD:
      skv::g_fused_bwd.store(value == 1 ? 3 : (value == 2 ? 1 : (value == 3 ? 2 : 0)), std::memory_order_relaxed);
      return SKV_OK;
    default:
      return SKV_ERR_UNSUPPORTED;
  }
}

int skv_resolve_impl(const skv_problem* p) {
  if (int e = validate(p)) return e;
  return resolve(*p);
}

size_t skv_scratch_bytes(const skv_problem* p, int op) {
  if (validate(p) != SKV_OK) return 0;
  const int impl = resolve(*p);
  if (impl == SKV_IMPL_SIMT) return simt_scratch_bytes(*p, op);
  if (impl != SKV_IMPL_TCGEN05) return 0;
  size_t need = tc_scratch_bytes(*p, op);
  if (p->impl == SKV_IMPL_AUTO) {
    // AUTO falls back to the CUDA-core kernels when a pointer or stride is not 16-byte aligned
    const size_t alt = simt_scratch_bytes(*p, op);
    if (alt > need) need = alt;
  }
  return need;
}

int skv_feature_forward(const skv_problem* p, const void* z, int64_t z_stride, const void* C, void* act_out,
                        int64_t act_stride, void* delta_out, int64_t delta_stride, void* scratch,
                        size_t scratch_bytes, int32_t* status, void* stream) {
  LaunchCtx c;
  if (int e = make_ctx(p, stream, status, &c)) return e;
  if (p->N == 0) return SKV_OK;
  if (!z || !C || !delta_out) return SKV_ERR_NULL;
  if (z_stride < p->h || delta_stride < p->r || (act_out && act_stride < p->h)) return SKV_ERR_SHAPE;
  const int impl = resolve(*p);
  if (impl < 0) return impl;
  if (impl == SKV_IMPL_TCGEN05) {
    if (!aligned(z, 16) || !aligned(C, 16) || !aligned(delta_out, 16) || (act_out && !aligned(act_out, 16)) ||
        z_stride % 8 || delta_stride % (p->delta_f32 ? 4 : 8) || (act_out && act_stride % 8)) {
      if (p->impl == SKV_IMPL_TCGEN05) return SKV_ERR_ALIGN;
    } else {
      if (!scratch || scratch_bytes < tc_scratch_bytes(*p, SKV_OP_FORWARD)) return SKV_ERR_SCRATCH;
      return tc_forward(c, z, z_stride, C, act_out, act_stride, delta_out, delta_stride, scratch, scratch_bytes);
    }
  }
  return simt_forward(c, z, z_stride, C, act_out, act_stride, delta_out, delta_stride);
}

int skv_feature_backward(const skv_problem* p, const void* z, int64_t z_stride, const void* C, const void* g_act,
                         int64_t gact_stride, const void* g_delta, int64_t gdelta_stride, void* dz,
                         int64_t dz_stride, float* dC_f32, void* dC_cast, void* scratch, size_t scratch_bytes,
                         int32_t* status, void* stream) {
  LaunchCtx c;
  if (int e = make_ctx(p, stream, status, &c)) return e;
  const size_t elems = (size_t)p->h * p->L * p->r;
  if (p->N == 0) {
    if (dC_f32 && cudaMemsetAsync(dC_f32, 0, elems * sizeof(float), c.stream) != cudaSuccess) return SKV_ERR_LAUNCH;
    if (dC_cast && cudaMemsetAsync(dC_cast, 0, elems * (p->dtype == SKV_BF16 ? 2 : 4), c.stream) != cudaSuccess)
      return SKV_ERR_LAUNCH;
    return SKV_OK;
  }
  if (!z || !C || !g_delta) return SKV_ERR_NULL;
  if (!dz && !dC_f32 && !dC_cast) return SKV_OK;
  if (z_stride < p->h || gdelta_stride < p->r || (g_act && gact_stride < p->h) || (dz && dz_stride < p->h))
    return SKV_ERR_SHAPE;
  const int impl = resolve(*p);
  if (impl < 0) return impl;
  const bool dz32 = p->dz_f32 && p->dtype == SKV_BF16;          // float32 dz of a bf16 problem: tcgen05 kernels only
  if (dz32 && impl != SKV_IMPL_TCGEN05) return SKV_ERR_UNSUPPORTED;
  if (impl == SKV_IMPL_TCGEN05) {
    if (!aligned(z, 16) || !aligned(C, 16) || !aligned(g_delta, 16) || (g_act && !aligned(g_act, 16)) ||
        (dz && !aligned(dz, 16)) || z_stride % 8 || gdelta_stride % 8 || (g_act && gact_stride % 8) ||
        (dz && dz_stride % (dz32 ? 4 : 8))) {
      if (p->impl == SKV_IMPL_TCGEN05 || dz32) return SKV_ERR_ALIGN;
    } else {
      if (!scratch || scratch_bytes < tc_scratch_bytes(*p, SKV_OP_BACKWARD)) return SKV_ERR_SCRATCH;
      return tc_backward(c, z, z_stride, C, g_act, gact_stride, g_delta, gdelta_stride, dz, dz_stride, dC_f32,
                         dC_cast, scratch, scratch_bytes);
    }
  }
  return simt_backward(c, z, z_stride, C, g_act, gact_stride, g_delta, gdelta_stride, dz, dz_stride, dC_f32,
                       dC_cast, scratch, scratch_bytes);
}

size_t skv_readout_scratch_bytes(const skv_problem* p, int64_t d_out) {
  if (validate(p) != SKV_OK || !tc::readout_eligible(*p, d_out)) return 0;
  skv_problem q = *p;
  q.delta_f32 = 0;
  return round256(skv_scratch_bytes(&q, SKV_OP_FORWARD)) + round256((size_t)p->N * tc::readout_delta_pitch(*p) * 2) +
         tc::readout_image_bytes(*p, d_out);
}

int skv_feature_readout_forward(const skv_problem* p, const void* z, int64_t z_stride, const void* C,
                                const void* w_out, int64_t w_stride, int64_t d_out, void* y, int64_t y_stride,
                                void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
  LaunchCtx c;
  if (int e = make_ctx(p, stream, status, &c)) return e;
  if (d_out < 1) return SKV_ERR_SHAPE;
  if (!tc::readout_eligible(*p, d_out)) return SKV_ERR_UNSUPPORTED;
  if (p->N == 0) return SKV_OK;
  if (!z || !C || !w_out || !y) return SKV_ERR_NULL;
  if (z_stride < p->h || w_stride < p->h + p->r || y_stride < d_out) return SKV_ERR_SHAPE;
  if (!aligned(z, 16) || !aligned(w_out, 16) || !aligned(y, 16) || z_stride % 8 || w_stride % 8 || y_stride % 8)
    return SKV_ERR_ALIGN;
  if (!scratch || !aligned(scratch, 256) || scratch_bytes < skv_readout_scratch_bytes(p, d_out)) return SKV_ERR_SCRATCH;
  skv_problem q = *p;
  q.delta_f32 = 0;
  const size_t fwd_bytes = round256(skv_scratch_bytes(&q, SKV_OP_FORWARD));
  uint8_t* base = static_cast<uint8_t*>(scratch);
  void* delta = base + fwd_bytes;
  const int64_t dp = tc::readout_delta_pitch(*p);
  void* wimg = base + fwd_bytes + round256((size_t)p->N * dp * 2);
  if (dp != p->r && cudaMemsetAsync(delta, 0, (size_t)p->N * dp * 2, c.stream) != cudaSuccess) return SKV_ERR_LAUNCH;
  if (int e = skv_feature_forward(&q, z, z_stride, C, nullptr, 0, delta, dp, scratch, fwd_bytes, status, stream))
    return e;
  return tc::readout(c, z, z_stride, delta, w_out, w_stride, d_out, y, y_stride, wimg);
}

int skv_knot_index(const skv_problem* p, const void* z, int64_t z_stride, int32_t* bins, void* stream) {
  LaunchCtx c;
  if (int e = make_ctx(p, stream, nullptr, &c)) return e;
  if (p->N == 0) return SKV_OK;
  if (!z || !bins) return SKV_ERR_NULL;
  if (z_stride < p->h) return SKV_ERR_SHAPE;
  return simt_knot_index(c, z, z_stride, bins);
}

}  // extern "C"
