// Shared device helpers of the spline-KV kernels: dtype access and the one
// knot-interval / B-spline-weight routine every kernel calls, so that all of
// them agree bit for bit on the interval index.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/splinekv_b200.h"

namespace skv {

// Grid constants prepared on the host once per call.
struct GridParams {
  float lo;      // grid_lo
  float scale;   // float32(G / (hi - lo))
  float Gf;      // (float)G
  float Gm1f;    // (float)(G - 1)
  int order;     // 2: quadratic B-spline (three weights per pair); 1: linear (two)
};

// Knot interval and local coordinate of one pre-activation value.
// Follows _b2_basis_and_bins of the reference
// (src/sparsespline_ffn/rl_spline_kv_reference.py:98-103): u = (z - lo) * scale in two separately
// rounded float32 operations, in_range = 0 <= u <= G, the clamp to [0, G-1], floor, tau.
// clamp_active = 0 <= u <= G-1 is where d clamp(u)/du = 1 (the mask of dz,
// src/sparsespline_ffn/kernels/flash_spline_feature_backward_ref.py:99-112).
struct Knot {
  int bin;
  float tau;
  bool in_range;
  bool clamp_active;
  uint32_t tbits;   // bit pattern of 2^23 + bin as float32: kKnotBias + bin
};

// Bit pattern of 2^23 as float32; Knot::tbits - kKnotBias is the interval index.
constexpr uint32_t kKnotBias = 0x4B000000u;

// The arithmetic is arranged for the instruction mix of the kernels that call it for every
// (token, key) pair, without changing any result:
//  * u is formed as fma(z - lo, scale, +0): the same rounding as the plain product, and a product
//    of -0 becomes +0, so that the two range tests are single unsigned comparisons of the bit
//    pattern (non-negative floats order like their bit patterns; negative values and NaN have
//    patterns above that of any grid bound);
//  * floor(u_c) is taken by adding 2^23 rounding down (u_c lies in [0, G-1], far below 2^22, so the
//    sum is exactly 2^23 + floor(u_c)) instead of a float -> int -> float round trip.
__device__ __forceinline__ Knot knot_of(float z, const GridParams& g) {
  Knot k;
  const float u = __fmaf_rn(__fsub_rn(z, g.lo), g.scale, 0.0f);
  const uint32_t ub = __float_as_uint(u);
  k.in_range = ub <= __float_as_uint(g.Gf);
  k.clamp_active = ub <= __float_as_uint(g.Gm1f);
  const float uc = fminf(fmaxf(u, 0.0f), g.Gm1f);   // NaN clamps to 0
  const float t = __fadd_rd(uc, 8388608.0f);
  k.tbits = __float_as_uint(t);
  k.bin = (int)(k.tbits & 0x007fffffu);
  k.tau = __fsub_rn(uc, __fsub_rn(t, 8388608.0f));  // exact, in [0, 1)
  return k;
}

// Forward weights B_0..B_2 (rl_spline_kv_reference.py:105-108), forward mask applied.
// order 1: the linear spline's 1 - tau and tau (rl_spline_kv_reference.py:139-141); B2 stays zero
// and its row must not be touched (it lies past the key's L = G + 1 rows).
__device__ __forceinline__ void basis_weights(const Knot& k, float& B0, float& B1, float& B2, int order = 2) {
  float t = k.tau, omt = 1.0f - t;
  float m = k.in_range ? 1.0f : 0.0f;
  if (order == 1) { B0 = omt * m; B1 = t * m; B2 = 0.0f; return; }
  B0 = 0.5f * omt * omt * m;
  B1 = 0.5f * (1.0f + 2.0f * t - 2.0f * t * t) * m;
  B2 = 0.5f * t * t * m;
}

// Derivative weights dB_k/dtau (flash_spline_feature_backward_ref.py:64-66), clamp mask applied.
__device__ __forceinline__ void basis_derivs(const Knot& k, float& d0, float& d1, float& d2, int order = 2) {
  float t = k.tau;
  float m = k.clamp_active ? 1.0f : 0.0f;
  if (order == 1) { d0 = -m; d1 = m; d2 = 0.0f; return; }
  d0 = -(1.0f - t) * m;
  d1 = (1.0f - 2.0f * t) * m;
  d2 = t * m;
}

// phi and phi' of the base path (rl_spline_kv_reference.py:78-85,
// flash_spline_feature_autograd.py:227-237).
// gelu is the exact erf form of torch.nn.functional.gelu; its derivative Phi(z) + z * pdf(z) is what
// autograd returns for it.
__device__ __forceinline__ float gelu_fwd(float z) { return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_grad(float z) {
  return 0.5f * (1.0f + erff(z * 0.70710678118654752f)) + z * expf(-0.5f * z * z) * 0.39894228040143268f;
}
__device__ __forceinline__ float act_fwd(float z, int act) {
  return act == SKV_ACT_RELU_SQ ? (z > 0.0f ? z * z : 0.0f) : act == SKV_ACT_GELU ? gelu_fwd(z) : z;
}
__device__ __forceinline__ float act_grad(float z, int act) {
  return act == SKV_ACT_RELU_SQ ? (z > 0.0f ? 2.0f * z : 0.0f) : act == SKV_ACT_GELU ? gelu_grad(z) : 1.0f;
}

template <typename T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(__ldg(p));
}
template <typename T> __device__ __forceinline__ void st_f32(T* p, float v);
template <> __device__ __forceinline__ void st_f32<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// Host-side count of kernel launches (reported by skv_kernel_launches()).
void note_launches(int n);

// Host-side launch context handed from the C ABI to the kernel families.
struct LaunchCtx {
  skv_problem p;
  GridParams g;
  int G;
  cudaStream_t stream;
  int32_t* status;
  int num_sms;
};

// CUDA-core kernel family (any N, h, L, r <= 256; bf16 or float32).
size_t simt_scratch_bytes(const skv_problem& p, int op);
int simt_forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
                 void* delta_out, int64_t ds);
int simt_backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
                  const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast,
                  void* scratch, size_t scratch_bytes);
int simt_knot_index(const LaunchCtx& c, const void* z, int64_t zs, int32_t* bins);

// tcgen05 kernel family (bf16, eligible shapes only).
bool tc_eligible(const skv_problem& p);
size_t tc_scratch_bytes(const skv_problem& p, int op);
int tc_forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
               void* delta_out, int64_t ds, void* scratch, size_t scratch_bytes);
int tc_backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
                const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast,
                void* scratch, size_t scratch_bytes);

}  // namespace skv
