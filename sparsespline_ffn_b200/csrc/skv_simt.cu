// CUDA-core kernels of the spline-KV feature operator: any N, h, L and r <= 256,
// bf16 or float32 I/O, float32 arithmetic.  They are the float32 tier of the
// library and the path for shapes the tcgen05 kernels do not cover.
//
// Mapping used by all three: one warp works on one (token, 32-key group) or
// (key, 32-token group) at a time; each lane evaluates the knot interval and
// B-spline weights of one (token, key) pair, then the warp walks the 32 pairs
// with the lanes spread over the r code channels, reading the code-table rows
// C[j, bin + k, :] from a float32 copy of the current key chunk in shared memory.
#include "skv_common.cuh"

namespace skv {
namespace {

constexpr int kWarp = 32;
constexpr int kMaxRIter = 8;          // r <= 256
constexpr unsigned kFull = 0xffffffffu;

__host__ __device__ inline int64_t cdiv64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------------
// Forward: grid.x = token blocks of TB tokens.  The CTA walks the keys in chunks of KCH keys,
// each warp owns TB/8 tokens and keeps their delta rows in shared memory.
// ---------------------------------------------------------------------------------------------
template <typename T, typename TD>
__global__ void __launch_bounds__(256)
simt_forward_kernel(const T* __restrict__ z, int64_t zs, const T* __restrict__ C,
                    T* __restrict__ act_out, int64_t as, TD* __restrict__ delta_out, int64_t ds,
                    int64_t N, int h, int L, int r, GridParams g, float lambda, int act, int TB, int KCH) {
  extern __shared__ float smem[];
  float* Cs = smem;                                   // [KCH][L][r]
  float* dacc = smem + (size_t)KCH * L * r;           // [TB][r]
  const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp, nwarps = blockDim.x / kWarp;
  const int64_t n0 = (int64_t)blockIdx.x * TB;
  const int riter = (r + kWarp - 1) / kWarp;
  const bool three = g.order != 1;                    // the linear spline has no third row

  for (int i = threadIdx.x; i < TB * r; i += blockDim.x) dacc[i] = 0.0f;

  for (int j0 = 0; j0 < h; j0 += KCH) {
    const int kc = min(KCH, h - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < kc * L * r; i += blockDim.x)
      Cs[i] = ld_f32<T>(C + (size_t)j0 * L * r + i);
    __syncthreads();

    for (int t = warp; t < TB; t += nwarps) {
      const int64_t n = n0 + t;
      if (n >= N) break;
      float acc[kMaxRIter];
#pragma unroll
      for (int ci = 0; ci < kMaxRIter; ++ci) acc[ci] = 0.0f;
      for (int jg = 0; jg < kc; jg += kWarp) {
        const int jl = jg + lane;
        int bin = 0;
        float B0 = 0.f, B1 = 0.f, B2 = 0.f;
        if (jl < kc) {
          float zz = ld_f32<T>(z + n * zs + j0 + jl);
          Knot k = knot_of(zz, g);
          basis_weights(k, B0, B1, B2, g.order);
          bin = k.bin;
          if (act_out) st_f32<T>(act_out + n * as + j0 + jl, act_fwd(zz, act));
        }
        const int cnt = min(kWarp, kc - jg);
        for (int q = 0; q < cnt; ++q) {
          const int b = __shfl_sync(kFull, bin, q);
          const float w0 = __shfl_sync(kFull, B0, q);
          const float w1 = __shfl_sync(kFull, B1, q);
          const float w2 = __shfl_sync(kFull, B2, q);
          const float* row = Cs + ((size_t)(jg + q) * L + b) * r;
#pragma unroll
          for (int ci = 0; ci < kMaxRIter; ++ci) {
            if (ci < riter) {
              const int c = ci * kWarp + lane;
              if (c < r) acc[ci] += w0 * row[c] + w1 * row[r + c] + (three ? w2 * row[2 * r + c] : 0.0f);
            }
          }
        }
      }
#pragma unroll
      for (int ci = 0; ci < kMaxRIter; ++ci) {
        if (ci < riter) {
          const int c = ci * kWarp + lane;
          if (c < r) dacc[t * r + c] += acc[ci];
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < TB * r; i += blockDim.x) {
    const int t = i / r, c = i % r;
    const int64_t n = n0 + t;
    if (n < N) st_f32<TD>(delta_out + n * ds + c, lambda * dacc[i]);
  }
}

// ---------------------------------------------------------------------------------------------
// dz: same walk as the forward; per pair the lanes hold g[n, c] * sum_k dB_k C[j, bin+k, c] for
// their channels, a butterfly transpose-reduce turns 32 such per-lane partials into one sum per
// lane (lane q ends up with the pair q), which then takes the base-path term and is stored.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
simt_dz_kernel(const T* __restrict__ z, int64_t zs, const T* __restrict__ C,
               const T* __restrict__ g_act, int64_t gas, const T* __restrict__ g_delta, int64_t gds,
               T* __restrict__ dz, int64_t dzs, int64_t N, int h, int L, int r, GridParams g,
               float lambda, int act, int TB, int KCH) {
  extern __shared__ float smem[];
  float* Cs = smem;                                   // [KCH][L][r]
  const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp, nwarps = blockDim.x / kWarp;
  const int64_t n0 = (int64_t)blockIdx.x * TB;
  const int riter = (r + kWarp - 1) / kWarp;
  const float coef = lambda * g.scale;
  const bool three = g.order != 1;

  for (int j0 = 0; j0 < h; j0 += KCH) {
    const int kc = min(KCH, h - j0);
    __syncthreads();
    for (int i = threadIdx.x; i < kc * L * r; i += blockDim.x)
      Cs[i] = ld_f32<T>(C + (size_t)j0 * L * r + i);
    __syncthreads();

    for (int t = warp; t < TB; t += nwarps) {
      const int64_t n = n0 + t;
      if (n >= N) break;
      float gd[kMaxRIter];
#pragma unroll
      for (int ci = 0; ci < kMaxRIter; ++ci) {
        const int c = ci * kWarp + lane;
        gd[ci] = (ci < riter && c < r) ? ld_f32<T>(g_delta + n * gds + c) : 0.0f;
      }
      for (int jg = 0; jg < kc; jg += kWarp) {
        const int jl = jg + lane;
        int bin = 0;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, zz = 0.f;
        if (jl < kc) {
          zz = ld_f32<T>(z + n * zs + j0 + jl);
          Knot k = knot_of(zz, g);
          basis_derivs(k, d0, d1, d2, g.order);
          bin = k.bin;
        }
        float v[kWarp];
        const int cnt = min(kWarp, kc - jg);
#pragma unroll
        for (int q = 0; q < kWarp; ++q) {
          float p = 0.0f;
          if (q < cnt) {
            const int b = __shfl_sync(kFull, bin, q);
            const float w0 = __shfl_sync(kFull, d0, q);
            const float w1 = __shfl_sync(kFull, d1, q);
            const float w2 = __shfl_sync(kFull, d2, q);
            const float* row = Cs + ((size_t)(jg + q) * L + b) * r;
#pragma unroll
            for (int ci = 0; ci < kMaxRIter; ++ci) {
              if (ci < riter) {
                const int c = ci * kWarp + lane;
                if (c < r) p += gd[ci] * (w0 * row[c] + w1 * row[r + c] + (three ? w2 * row[2 * r + c] : 0.0f));
              }
            }
          }
          v[q] = p;
        }
        // butterfly transpose-reduce: afterwards v[0] on lane q is the sum over lanes of v[q]
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
#pragma unroll
          for (int i = 0; i < s; ++i) {
            const bool up = (lane & s) != 0;
            const float send = up ? v[i] : v[i + s];
            const float keep = up ? v[i + s] : v[i];
            v[i] = keep + __shfl_xor_sync(kFull, send, s);
          }
        }
        if (jl < kc) {
          float out = coef * v[0];
          if (g_act) out += ld_f32<T>(g_act + n * gas + j0 + jl) * act_grad(zz, act);
          st_f32<T>(dz + n * dzs + j0 + jl, out);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// dC partials: grid = (key groups of KD keys, token splits).  One warp per key; the warp owns a
// private [L][r] float32 accumulator in shared memory, so no atomics are needed and the sum
// order is fixed.  z and g_delta tiles of TT tokens are staged in shared memory.
// part[split][h][L][r] is written; simt_dc_reduce_kernel sums the splits.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512)
simt_dc_partial_kernel(const T* __restrict__ z, int64_t zs, const T* __restrict__ g_delta, int64_t gds,
                       float* __restrict__ part, int64_t N, int h, int L, int r, GridParams g,
                       int KD, int TT, int64_t tokens_per_split) {
  extern __shared__ float smem[];
  float* acc = smem;                                  // [KD][L][r]
  float* gs = acc + (size_t)KD * L * r;               // [TT][r]
  float* zt = gs + (size_t)TT * r;                    // [TT][KD]
  const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
  const int j0 = blockIdx.x * KD;
  const int kd = min(KD, h - j0);
  const int64_t nb = (int64_t)blockIdx.y * tokens_per_split;
  const int64_t ne = min(N, nb + tokens_per_split);
  const int riter = (r + kWarp - 1) / kWarp;

  const bool three = g.order != 1;
  for (int i = threadIdx.x; i < KD * L * r; i += blockDim.x) acc[i] = 0.0f;
  float* my = acc + (size_t)warp * L * r;

  for (int64_t t0 = nb; t0 < ne; t0 += TT) {
    const int tt = (int)min((int64_t)TT, ne - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < tt * r; i += blockDim.x)
      gs[i] = ld_f32<T>(g_delta + (t0 + i / r) * gds + i % r);
    for (int i = threadIdx.x; i < tt * KD; i += blockDim.x) {
      const int t = i / KD, k = i % KD;
      zt[i] = k < kd ? ld_f32<T>(z + (t0 + t) * zs + j0 + k) : 0.0f;
    }
    __syncthreads();
    if (warp < kd) {
      for (int tg = 0; tg < tt; tg += kWarp) {
        int bin = 0;
        float B0 = 0.f, B1 = 0.f, B2 = 0.f;
        if (tg + lane < tt) {
          Knot k = knot_of(zt[(tg + lane) * KD + warp], g);
          basis_weights(k, B0, B1, B2, g.order);
          bin = k.bin;
        }
        const int cnt = min(kWarp, tt - tg);
        for (int q = 0; q < cnt; ++q) {
          const int b = __shfl_sync(kFull, bin, q);
          const float w0 = __shfl_sync(kFull, B0, q);
          const float w1 = __shfl_sync(kFull, B1, q);
          const float w2 = __shfl_sync(kFull, B2, q);
          float* row = my + (size_t)b * r;
          const float* gr = gs + (size_t)(tg + q) * r;
          for (int ci = 0; ci < riter; ++ci) {
            const int c = ci * kWarp + lane;
            if (c < r) {
              const float gv = gr[c];
              row[c] += w0 * gv;
              row[r + c] += w1 * gv;
              if (three) row[2 * r + c] += w2 * gv;
            }
          }
        }
      }
    }
  }
  __syncthreads();
  float* dst = part + ((size_t)blockIdx.y * h + j0) * L * r;
  for (int i = threadIdx.x; i < kd * L * r; i += blockDim.x) dst[i] = acc[i];
}

template <typename T>
__global__ void simt_dc_reduce_kernel(const float* __restrict__ part, int splits, size_t elems, float lambda,
                                      float* __restrict__ dC, T* __restrict__ dC_cast) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += (size_t)gridDim.x * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += part[(size_t)k * elems + i];
    s *= lambda;
    if (dC) dC[i] = s;
    if (dC_cast) st_f32<T>(dC_cast + i, s);
  }
}

template <typename T>
__global__ void simt_knot_index_kernel(const T* __restrict__ z, int64_t zs, int64_t N, int h, GridParams g,
                                       int32_t* __restrict__ bins) {
  const int64_t total = N * (int64_t)h;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i / h;
    const int j = (int)(i % h);
    bins[i] = knot_of(ld_f32<T>(z + n * zs + j), g).bin;
  }
}

constexpr size_t kSmemBudget = 160 * 1024;

struct FwdPlan { int TB, KCH; size_t smem; };
FwdPlan plan_token_major(const skv_problem& p, bool with_dacc) {
  FwdPlan f;
  f.TB = 128;
  const size_t per_key = (size_t)p.L * p.r * sizeof(float);
  const size_t dacc = with_dacc ? (size_t)f.TB * p.r * sizeof(float) : 0;
  size_t kch = (kSmemBudget - dacc) / per_key;
  if (kch >= 32) kch = kch / 32 * 32;
  if (kch > 64) kch = 64;
  if (kch > (size_t)p.h) kch = p.h;
  if (kch < 1) kch = 1;
  f.KCH = (int)kch;
  f.smem = kch * per_key + dacc;
  return f;
}

struct DcPlan { int KD, TT, splits; int64_t tokens_per_split; size_t smem; };
DcPlan plan_dc(const skv_problem& p, int num_sms) {
  DcPlan d;
  const size_t per_key = (size_t)p.L * p.r * sizeof(float);
  d.TT = 64;
  int kd = 16;
  while (kd > 1 && kd * per_key + (size_t)d.TT * (p.r + kd) * sizeof(float) > kSmemBudget) kd /= 2;
  d.KD = kd;
  d.smem = kd * per_key + (size_t)d.TT * (p.r + kd) * sizeof(float);
  const int64_t groups = cdiv64(p.h, kd);
  int64_t splits = cdiv64(2 * (int64_t)num_sms, groups);
  const int64_t max_splits = cdiv64(p.N, 256);
  if (splits > max_splits) splits = max_splits;
  if (splits > 16) splits = 16;
  if (splits < 1) splits = 1;
  d.tokens_per_split = cdiv64(cdiv64(p.N, splits), d.TT) * d.TT;
  if (d.tokens_per_split < d.TT) d.tokens_per_split = d.TT;
  d.splits = (int)cdiv64(p.N, d.tokens_per_split);
  if (d.splits < 1) d.splits = 1;
  return d;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
      cudaGetLastError();
      return SKV_ERR_LAUNCH;
    }
  }
  return SKV_OK;
}

template <typename T, typename TD>
int forward_t(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
              void* delta_out, int64_t ds) {
  const skv_problem& p = c.p;
  FwdPlan f = plan_token_major(p, true);
  if (int e = set_smem(simt_forward_kernel<T, TD>, f.smem)) return e;
  const unsigned grid = (unsigned)cdiv64(p.N, f.TB);
  simt_forward_kernel<T, TD><<<grid, 256, f.smem, c.stream>>>(
      (const T*)z, zs, (const T*)C, (T*)act_out, as, (TD*)delta_out, ds, p.N, p.h, p.L, p.r, c.g,
      p.lambda_scale, p.activation, f.TB, f.KCH);
  note_launches(1);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_LAUNCH;
}

template <typename T>
int backward_t(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
               const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast,
               void* scratch, size_t scratch_bytes) {
  const skv_problem& p = c.p;
  if (dz) {
    FwdPlan f = plan_token_major(p, false);
    if (int e = set_smem(simt_dz_kernel<T>, f.smem)) return e;
    const unsigned grid = (unsigned)cdiv64(p.N, f.TB);
    simt_dz_kernel<T><<<grid, 256, f.smem, c.stream>>>(
        (const T*)z, zs, (const T*)C, (const T*)g_act, gas, (const T*)g_delta, gds, (T*)dz, dzs, p.N, p.h, p.L,
        p.r, c.g, p.lambda_scale, p.activation, f.TB, f.KCH);
    note_launches(1);
    if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
  }
  if (dC || dC_cast) {
    DcPlan d = plan_dc(p, c.num_sms);
    const size_t elems = (size_t)p.h * p.L * p.r;
    if (!scratch || scratch_bytes < (size_t)d.splits * elems * sizeof(float)) return SKV_ERR_SCRATCH;
    if (int e = set_smem(simt_dc_partial_kernel<T>, d.smem)) return e;
    dim3 grid((unsigned)cdiv64(p.h, d.KD), (unsigned)d.splits);
    simt_dc_partial_kernel<T><<<grid, d.KD * kWarp, d.smem, c.stream>>>(
        (const T*)z, zs, (const T*)g_delta, gds, (float*)scratch, p.N, p.h, p.L, p.r, c.g, d.KD, d.TT,
        d.tokens_per_split);
    if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
    const unsigned rgrid = (unsigned)((elems + 255) / 256 < 4096 ? (elems + 255) / 256 : 4096);
    simt_dc_reduce_kernel<T><<<rgrid, 256, 0, c.stream>>>((const float*)scratch, d.splits, elems,
                                                           p.lambda_scale, dC, (T*)dC_cast);
    note_launches(2);
    if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
  }
  return SKV_OK;
}

}  // namespace

size_t simt_scratch_bytes(const skv_problem& p, int op) {
  if (op != SKV_OP_BACKWARD) return 0;
  // independent of the SM count actually present: sized for the largest split count plan_dc can pick
  DcPlan d = plan_dc(p, 148);
  int splits = d.splits;
  DcPlan d2 = plan_dc(p, 256);
  if (d2.splits > splits) splits = d2.splits;
  return (size_t)splits * p.h * p.L * p.r * sizeof(float);
}

int simt_forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
                 void* delta_out, int64_t ds) {
  if (c.p.dtype == SKV_F32) return forward_t<float, float>(c, z, zs, C, act_out, as, delta_out, ds);
  return c.p.delta_f32 ? forward_t<__nv_bfloat16, float>(c, z, zs, C, act_out, as, delta_out, ds)
                       : forward_t<__nv_bfloat16, __nv_bfloat16>(c, z, zs, C, act_out, as, delta_out, ds);
}

int simt_backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
                  const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast,
                  void* scratch, size_t scratch_bytes) {
  return c.p.dtype == SKV_BF16
             ? backward_t<__nv_bfloat16>(c, z, zs, C, g_act, gas, g_delta, gds, dz, dzs, dC, dC_cast, scratch,
                                         scratch_bytes)
             : backward_t<float>(c, z, zs, C, g_act, gas, g_delta, gds, dz, dzs, dC, dC_cast, scratch,
                                 scratch_bytes);
}

int simt_knot_index(const LaunchCtx& c, const void* z, int64_t zs, int32_t* bins) {
  const int64_t total = c.p.N * (int64_t)c.p.h;
  const unsigned grid = (unsigned)(cdiv64(total, 256) < 8192 ? cdiv64(total, 256) : 8192);
  if (c.p.dtype == SKV_BF16)
    simt_knot_index_kernel<__nv_bfloat16><<<grid, 256, 0, c.stream>>>((const __nv_bfloat16*)z, zs, c.p.N, c.p.h,
                                                                       c.g, bins);
  else
    simt_knot_index_kernel<float><<<grid, 256, 0, c.stream>>>((const float*)z, zs, c.p.N, c.p.h, c.g, bins);
  note_launches(1);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_LAUNCH;
}

}  // namespace skv
