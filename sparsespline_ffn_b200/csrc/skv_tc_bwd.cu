// tcgen05 backward of the spline-KV feature operator (bf16 I/O).
//
// dz kernel (token-major, like the forward):
//   S[n, (j,m)] = sum_c g[n,c] * T[j,m,c]   on the tensor cores (M = 128 tokens, N = 8L, K = r)
//   where T is the code table transformed along the knot axis so that the three-of-L selection
//   becomes a dense weighted sum with one saturating add per column:
//       T[j,0]   = C[j,1] - C[j,0]
//       T[j,m+1] = C[j,m] - 2 C[j,m+1] + C[j,m+2]      (m = 0..G-1),   T[j,L-1] = 0
//       dz_spline[n,j] = scale * 1[0 <= u <= G-1] * ( S[n,(j,0)] + sum_m sat(u_c - m) * S[n,(j,m+1)] )
//   (sat(u_c - m) is 1 below the token's knot interval, tau inside it and 0 above, which telescopes
//   to -(1-tau) C[bin] + (1-2tau) C[bin+1] + tau C[bin+2], the B-spline derivative weights.)
//   One thread per token reads its S row from tensor memory, adds the base-path term
//   g_a * phi'(z) and stores dz in bf16.
//
// dC kernel (key-major):
//   dC[(j,b), c] = sum_n Phi[n,(j,b)] * g[n,c]  (M = knot rows of a key chunk, N = r, K = tokens)
//   A CTA owns a slab of keys, keeps the slab's accumulators in tensor memory and streams
//   128-token tiles: two producer groups alternate, each building the f16 Phi tile of its token
//   tile for one key chunk in its own shared-memory stage while the MMAs of the other run.
//   The token range is split over CTAs; a reduce kernel sums the splits in a fixed order.
//
// The upstream gradient is converted once per call to f16, multiplied by a power of two chosen
// from its largest magnitude so that small gradients do not underflow; the inverse factor is
// applied to the float32 results.
#include "skv_tc_common.cuh"

namespace skv {
namespace tc {

size_t cimg_bytes(const skv_problem& p);
bool fwd_eligible(const skv_problem& p);


namespace {

constexpr int kChunkKeys = 8;
constexpr int kPlanSMs = 148;
constexpr size_t kSmemMax = 227 * 1024;

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// g [N][r] bf16 -> scaled f16 image, per 128-token tile the 8x8 core matrices (token rows of 16
// bytes) at ((cg * 16 + tg) * 128) bytes; rows past N are zero.
__global__ void tc_pack_g_kernel(const __nv_bfloat16* __restrict__ g, int64_t gds, int64_t N, int r, int64_t tiles,
                                 const uint32_t* __restrict__ amax_bits, __half* __restrict__ img) {
  float scale, inv;
  pow2_scales(*amax_bits, scale, inv);
  const int cgs = r / 8;
  const int64_t pieces = tiles * 128 * cgs;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (int64_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cgs);
    const int64_t n = i / cgs;
    uint32_t o[4] = {0, 0, 0, 0};
    if (n < N) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(g + n * gds + cg * 8));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) o[q] = pack_h2(bf_lo(w[q]) * scale, bf_hi(w[q]) * scale);
    }
    const int64_t tile = n >> 7;
    const int t = (int)(n & 127);
    __half* dst = img + (size_t)tile * 128 * r + ((size_t)cg * 16 + (t >> 3)) * 64 + (t & 7) * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Transformed table T (see the file header) as an f16 image in the same core-matrix layout as the
// forward's code-table image, with every key padded to LP (a multiple of 8) rows of which rows
// L-1.. are zero: per 8-key chunk the [8*LP x r] tile as 8x8 core matrices, core (rowg, cg) at
// ((rowg * r/8 + cg) * 128) bytes.
__global__ void tc_pack_t_kernel(const __nv_bfloat16* __restrict__ C, __half* __restrict__ img, int h, int L, int LP,
                                 int r, const uint32_t* __restrict__ amax_bits) {
  float cscale, cinv;
  pow2_scales(amax_bits[kAmaxC], cscale, cinv);
  const int rows_per_chunk = kChunkKeys * LP;
  const int cgs = r / 8;
  const size_t pieces = (size_t)h * LP * cgs;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (size_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cgs);
    const size_t rowg = i / cgs;
    const int j = (int)(rowg / LP), m = (int)(rowg % LP);
    const __nv_bfloat16* base = C + (size_t)j * L * r + cg * 8;
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (m == 0) v[q] = __bfloat162float(base[r + q]) - __bfloat162float(base[q]);
      else if (m >= L - 1) v[q] = 0.0f;
      else
        v[q] = __bfloat162float(base[(size_t)(m - 1) * r + q]) - 2.0f * __bfloat162float(base[(size_t)m * r + q]) +
               __bfloat162float(base[(size_t)(m + 1) * r + q]);
      v[q] *= cscale;                                   // a power of two: exact
    }
    const int chunk = (int)(rowg / rows_per_chunk);
    const int k = (int)(rowg % rows_per_chunk);
    __half* dst = img + (size_t)chunk * rows_per_chunk * r + ((size_t)(k >> 3) * cgs + cg) * 64 + (k & 7) * 8;
    *reinterpret_cast<uint4*>(dst) =
        make_uint4(pack_h2(v[0], v[1]), pack_h2(v[2], v[3]), pack_h2(v[4], v[5]), pack_h2(v[6], v[7]));
  }
}

// =================================================================================================
// dz
// =================================================================================================
struct DzParams {
  const __nv_bfloat16* z;
  int64_t zs;
  const __nv_bfloat16* g_act;
  int64_t gas;
  __nv_bfloat16* dz;
  int64_t dzs;
  const __half* gimg;
  const __half* timg;
  const uint32_t* amax_bits;
  int64_t N;
  int h, L, r;
  GridParams g;
  int act;
  float coef;                // lambda * scale
  int chunks_total, chunks_per_split;
  int tstages;               // depth of the transformed-table ring (2..kTStages)
  int dz_f32;                // dz is float32 [N][dzs] instead of bf16
  int32_t* status;
  long long wait_cycles;     // limit of every bounded wait, in clock cycles
};


// Tensor-memory loads of one key's S columns: the first NC of its LB blocks of 8 float32 columns of
// this warp's lanes (the padding columns are never read: the kernel's time follows the bytes it moves
// out of tensor memory, 4 * NC per pair).  The loads are issued without waiting; tmem_wait_key waits
// for all outstanding loads and ties the destination registers to the wait so that no use can be
// scheduled ahead of it.
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r);
template <> __device__ __forceinline__ void tmem_ld_cols<8>(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_cols<4>(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_cols<2>(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_cols<1>(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r[0]) : "r"(taddr) : "memory");
}
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// All 8 * LB columns of the key, in as few instructions as possible (a load instruction costs more
// than the columns it moves: loading only the NC useful columns as 8 + 8 + 4 + 1 was slower, 1.16 ms
// against 1.11 ms at the d20 shape).
template <int LB, int NC>
__device__ __forceinline__ void tmem_ld_key(uint32_t taddr, uint32_t (&r)[LB][8]) {
  uint32_t* flat = &r[0][0];
  int o = 0;
#pragma unroll
  for (int i = 0; i < LB / 2; ++i) { tmem_ld_cols<16>(taddr + (uint32_t)o, flat + o); o += 16; }
  if constexpr ((LB & 1) != 0) tmem_ld_cols<8>(taddr + (uint32_t)o, flat + o);
}
template <int LB, int NC>
__device__ __forceinline__ void tmem_wait_key(uint32_t (&r)[LB][8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int blk = 0; blk < LB; ++blk)
#pragma unroll
    for (int i = 0; i < 8; ++i) asm volatile("" : "+r"(r[blk][i]) : : "memory");
}

// S_0 + sum_m sat(uc - m) * S_{m+1} over the first NC of the 8*LB columns of one key.  Columns
// L-1 and up are padding (zero rows of the table image, and their weight sat(uc - m) is zero as
// well since uc <= G-1 < m); with NC = L-1 known at compile time they cost nothing.
// Columns are taken in aligned pairs with the packed two-wide float32 FMA of sm_100
// (fma.rn.f32x2): weight 1 for column 0, sat(uc - (m-1)) for column m.
template <int LB, int NC>
__device__ __forceinline__ float dz_key_sum(const uint32_t (&r)[LB][8], float uc) {
  unsigned long long acc2 = 0ull;                     // (0.0f, 0.0f)
  float tail = 0.0f;
#pragma unroll
  for (int blk = 0; blk < LB; ++blk) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const int m = blk * 8 + i;
      if (m >= NC) continue;
      const float w0 = m == 0 ? 1.0f : __saturatef(uc - (float)(m - 1));
      if (m + 1 >= NC) {                              // last column of an odd count
        tail = w0 * __uint_as_float(r[blk][i]);
        continue;
      }
      const float w1 = __saturatef(uc - (float)m);
      unsigned long long w2, s2;
      asm("mov.b64 %0, {%1, %2};" : "=l"(w2) : "f"(w0), "f"(w1));
      asm("mov.b64 %0, {%1, %2};" : "=l"(s2) : "r"(r[blk][i]), "r"(r[blk][i + 1]));
      asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2) : "l"(w2), "l"(s2));
    }
  }
  float a0, a1;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc2));
  return (a0 + a1) + tail;
}

constexpr int kTStages = 4;

// RELU: the base path is ReLU^2 (compile-time, so that the code of the other activations stays
// out of the hot loop); otherwise P.act (identity or gelu) is evaluated at run time.
template <int GROUPS, int LB, int NC, bool RELU>
__global__ void __launch_bounds__(128 * GROUPS + 64, 1) tc_dz_kernel(const DzParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int r = P.r;
  constexpr int LP = 8 * LB;                                         // padded knot columns per key
  const uint32_t g_bytes = (uint32_t)(128 * r * 2);
  const uint32_t t_bytes = (uint32_t)(kChunkKeys * LP * r * 2);
  constexpr uint32_t ncols = (uint32_t)(kChunkKeys * LP);            // S columns per group
  uint8_t* g_base = smem;                                             // [group][g_bytes]
  uint8_t* t_base = smem + (size_t)GROUPS * g_bytes;                  // [kTStages][t_bytes]
  const int TS = P.tstages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(t_base + (size_t)TS * t_bytes);
  uint64_t* gfull = bars;                    // [1]
  uint64_t* tfull = gfull + 1;               // [kTStages]
  uint64_t* tempty = tfull + kTStages;       // [kTStages]
  uint64_t* sfull = tempty + kTStages;       // [GROUPS]  MMA -> consumers
  uint64_t* sempty = sfull + GROUPS;         // [GROUPS]  consumers -> MMA
  uint64_t* done = sempty + GROUPS;          // [1]       all MMAs of this CTA complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutDz, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk_begin = blockIdx.y * P.chunks_per_split;
  const int nch = min(P.chunks_per_split, P.chunks_total - chunk_begin);
  const int64_t tile_base = (int64_t)blockIdx.x * (128 * GROUPS);
  uint32_t tmem_cols = 32;
  while (tmem_cols < GROUPS * ncols) tmem_cols <<= 1;

  if (tid == 0) {
    mbar_init(gfull, 1);
    for (int i = 0; i < kTStages; ++i) { mbar_init(tfull + i, 1); mbar_init(tempty + i, 1); }
    for (int i = 0; i < GROUPS; ++i) { mbar_init(sfull + i, 1); mbar_init(sempty + i, 4); }
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 4 * GROUPS) tmem_alloc(tmem_slot, tmem_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4 * GROUPS) {
    // ------------------------------------------------------------------ one thread per token
    const int grp = warp >> 2;
    const int t = tid & 127;
    const int64_t n = tile_base + grp * 128 + t;
    const bool valid = n < P.N;
    const int64_t nn = valid ? n : 0;
    const __nv_bfloat16* zrow = P.z + nn * P.zs + (int64_t)chunk_begin * kChunkKeys;
    const __nv_bfloat16* garow = P.g_act ? P.g_act + nn * P.gas + (int64_t)chunk_begin * kChunkKeys : nullptr;
    __nv_bfloat16* dzrow = P.dz + nn * P.dzs + (int64_t)chunk_begin * kChunkKeys;
    float gscale, ginv;
    pow2_scales(*P.amax_bits, gscale, ginv);
    float cscale, cinv;
    pow2_scales(P.amax_bits[kAmaxC], cscale, cinv);
    const float coef = P.coef * ginv * cinv;
    const int act = P.act;
    const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)grp * ncols;
    uint4 znext = valid && nch > 0 ? __ldg(reinterpret_cast<const uint4*>(zrow)) : make_uint4(0, 0, 0, 0);
    uint4 ganext = valid && nch > 0 && garow ? __ldg(reinterpret_cast<const uint4*>(garow)) : make_uint4(0, 0, 0, 0);

    for (int ci = 0; ci < nch; ++ci) {
      const uint4 zc = znext, gac = ganext;
      if (ci + 1 < nch && valid) {
        znext = __ldg(reinterpret_cast<const uint4*>(zrow + (ci + 1) * kChunkKeys));
        if (garow) ganext = __ldg(reinterpret_cast<const uint4*>(garow + (ci + 1) * kChunkKeys));
      }
      const uint32_t zw[4] = {zc.x, zc.y, zc.z, zc.w};
      const uint32_t gw[4] = {gac.x, gac.y, gac.z, gac.w};
      uint32_t bufa[LB][8], bufb[LB][8];
      float outv[kChunkKeys];
      mbar_wait(sfull + grp, (uint32_t)ci & 1u, wc);
      tc_fence_after();
      tmem_ld_key<LB, NC>(trow, bufa);
#pragma unroll
      for (int q = 0; q < kChunkKeys; ++q) {
        // the loads of key q are in flight; wait, start the loads of key q+1, then do key q's math
        if (q & 1) tmem_wait_key<LB, NC>(bufb); else tmem_wait_key<LB, NC>(bufa);
        if (q + 1 < kChunkKeys) {
          if (q & 1) tmem_ld_key<LB, NC>(trow + (uint32_t)((q + 1) * LP), bufa);
          else tmem_ld_key<LB, NC>(trow + (uint32_t)((q + 1) * LP), bufb);
        }
        const float zz = (q & 1) ? bf_hi(zw[q >> 1]) : bf_lo(zw[q >> 1]);
        // same u and the same single-comparison range test as knot_of
        const float u = __fmaf_rn(__fsub_rn(zz, P.g.lo), P.g.scale, 0.0f);
        const bool active = __float_as_uint(u) <= __float_as_uint(P.g.Gm1f);
        const float uc = fminf(fmaxf(u, 0.0f), P.g.Gm1f);
        const float acc = (q & 1) ? dz_key_sum<LB, NC>(bufb, uc) : dz_key_sum<LB, NC>(bufa, uc);
        float o = active ? coef * acc : 0.0f;
        if (garow) {
          const float ga = (q & 1) ? bf_hi(gw[q >> 1]) : bf_lo(gw[q >> 1]);
          const float dphi = RELU ? 2.0f * fmaxf(zz, 0.0f) : act_grad(zz, act);
          o = fmaf(ga, dphi, o);
        }
        outv[q] = o;
      }
      // (Handing the S columns back two keys earlier, with the loads running two keys ahead in a third
      // register buffer, was measured slower: 1.14 ms against 1.11 ms at the d20 shape.)
      tc_fence_before();
      mbar_arrive_warp(sempty + grp);
      if (valid) {
        if (P.dz_f32) {
          float* o = reinterpret_cast<float*>(P.dz) + nn * P.dzs + (int64_t)(chunk_begin + ci) * kChunkKeys;
          *reinterpret_cast<float4*>(o) = make_float4(outv[0], outv[1], outv[2], outv[3]);
          *reinterpret_cast<float4*>(o + 4) = make_float4(outv[4], outv[5], outv[6], outv[7]);
        } else {
          *reinterpret_cast<uint4*>(dzrow + ci * kChunkKeys) =
              make_uint4(pack_bf2(outv[0], outv[1]), pack_bf2(outv[2], outv[3]), pack_bf2(outv[4], outv[5]),
                         pack_bf2(outv[6], outv[7]));
        }
      }
    }
  } else if (warp == 4 * GROUPS) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      mbar_wait(gfull, 0, wc);
      const uint32_t rb = (uint32_t)(r / 8) * 128u;          // bytes between 8-row groups of the T image
      const uint32_t a_hi = desc_hi(128u), b_hi = desc_hi(rb);
      // The groups are served in a fixed order.  (Serving whichever group has released its S columns
      // first, by polling both, was measured slower: 1.32 ms against 1.21 ms at the d20 shape.)
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % TS;
        bool drain = mbar_wait(tfull + s, (uint32_t)(ci / TS) & 1u, wc);
        const uint32_t b_addr = smem_u32(t_base + (size_t)s * t_bytes);
        for (int grp = 0; grp < GROUPS && !drain; ++grp) {
          if (ci > 0) drain = mbar_wait(sempty + grp, (uint32_t)(ci - 1) & 1u, wc);
          if (drain) break;                          // draining: issue nothing more
          tc_fence_after();
          const uint32_t a_lo0 = desc_lo(smem_u32(g_base + (size_t)grp * g_bytes), 2048u);
          for (uint32_t c0 = 0; c0 < ncols; c0 += 256) {
            const uint32_t npiece = min(256u, ncols - c0);
            const uint32_t idesc = instr_desc(0, 0, 0, 0, 128, (int)npiece);
            uint32_t a_lo = a_lo0;
            uint32_t b_lo = desc_lo(b_addr + (c0 / 8) * rb, 128u);
            const uint32_t d_addr = tmem_base + (uint32_t)grp * ncols + c0;
            for (int ks = 0; ks < r / 16; ++ks) {
              umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, ks > 0 ? 1u : 0u);
              a_lo += 4096u >> 4;
              b_lo += 256u >> 4;
            }
          }
          umma_commit(sfull + grp);
        }
        if (drain) break;
        umma_commit(tempty + s);
      }
      umma_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      mbar_arrive_expect_tx(gfull, GROUPS * g_bytes);
      for (int grp = 0; grp < GROUPS; ++grp)
        bulk_g2s(g_base + (size_t)grp * g_bytes,
                 reinterpret_cast<const uint8_t*>(P.gimg) + (size_t)(blockIdx.x * GROUPS + grp) * g_bytes, g_bytes,
                 gfull);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(P.timg) + (size_t)chunk_begin * t_bytes;
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % TS;
        if (ci >= TS)
          mbar_wait(tempty + s, (uint32_t)((ci / TS) - 1) & 1u, wc);
        if (*abort_flag) break;
        mbar_arrive_expect_tx(tfull + s, t_bytes);
        bulk_g2s(t_base + (size_t)s * t_bytes, src + (size_t)ci * t_bytes, t_bytes, tfull + s);
      }
      if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4 * GROUPS) {
    mbar_wait_drain(done, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, tmem_cols);
  }
}

// =================================================================================================
// dC
// =================================================================================================
struct DcParams {
  const __nv_bfloat16* z;
  int64_t zs;
  const __half* gimg;
  float* part;               // [splits][h*L][r]
  int64_t N;
  int h, L, r;
  GridParams g;
  int LR;                    // knot rows per key in the Phi^T tile: L rounded up to even (pad row zero)
  int kch;                   // keys per chunk (8 or 16)
  int mtiles;                // 128-row MMA tiles per chunk
  int slab_chunks;           // chunks per CTA slab
  int64_t tiles_per_split;   // 128-token tiles per token split
  int64_t tiles_total;
  int32_t* status;
  long long wait_cycles;     // limit of every bounded wait, in clock cycles
};

// KCH = keys per chunk.  Two producer groups of 128 threads (thread = token of the group's tile).
template <int KCH, int HLC>
__global__ void __launch_bounds__(256 + 64, 1) tc_dc_kernel(const DcParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int L = P.L, LR = HLC ? 2 * HLC : P.LR, r = P.r;
  const uint32_t phi_bytes = (uint32_t)P.mtiles * 16u * 2048u;     // [m groups][16 token groups][8 tok][8 m]
  const uint32_t g_bytes = (uint32_t)(128 * r * 2);
  uint8_t* phi_base = smem;                                         // [2][phi_bytes]
  uint8_t* g_base = smem + 2 * (size_t)phi_bytes;                   // [2][g_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(g_base + 2 * (size_t)g_bytes);
  uint64_t* pfull = bars;          // [2] producers -> MMA
  uint64_t* pempty = pfull + 2;    // [2][3] MMA -> producers, per 128-row tile
  uint64_t* gfull = pempty + 6;    // [2] TMA -> MMA
  uint64_t* gempty = gfull + 2;    // [2] MMA -> TMA
  uint64_t* done = gempty + 2;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutDc, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rows = KCH * LR;                                         // (padded) knot rows per chunk
  const int key0 = blockIdx.x * P.slab_chunks * KCH;
  const int nchunks = min(P.slab_chunks, (P.h - key0 + KCH - 1) / KCH);
  const int64_t tile_begin = (int64_t)blockIdx.y * P.tiles_per_split;
  const int ntiles = (int)min(P.tiles_per_split, P.tiles_total - tile_begin);
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)(P.slab_chunks * P.mtiles * r)) tmem_cols <<= 1;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(pfull + i, 4);
      mbar_init(gfull + i, 1);
      mbar_init(gempty + i, 1);
    }
    for (int i = 0; i < 6; ++i) mbar_init(pempty + i, 1);
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  {
    uint4* p = reinterpret_cast<uint4*>(phi_base);
    const uint32_t n16 = 2 * phi_bytes / 16;
    for (uint32_t i = tid; i < n16; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == 8) tmem_alloc(tmem_slot, tmem_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // ------------------------------------------------------------------ producers
    const int pg = warp >> 2;
    const int t = tid & 127;
    const uint32_t t_off = (uint32_t)(t & 7) * 16u + (uint32_t)(t >> 3) * 128u;
    const uint32_t row = smem_u32(phi_base + (size_t)pg * phi_bytes) + t_off;
    const uint32_t halfL = (uint32_t)LR >> 1;
    uint32_t saved[KCH];
#pragma unroll
    for (int i = 0; i < KCH; ++i) saved[i] = 0;
    bool have_saved = false;
    int use = 0;                                     // how often this group's stage has been filled
    for (int ti = pg; ti < ntiles; ti += 2) {
      const int64_t n = (tile_begin + ti) * 128 + t;
      const bool valid = n < P.N;
      const __nv_bfloat16* zrow = P.z + (valid ? n : 0) * P.zs + key0;
      // pre-activations of the chunk after this one are requested before this one is processed
      uint4 znext[KCH / 8];
#pragma unroll
      for (int i = 0; i < KCH / 8; ++i)
        znext[i] = valid && key0 + i * 8 < P.h ? __ldg(reinterpret_cast<const uint4*>(zrow + i * 8)) : make_uint4(0, 0, 0, 0);
      for (int ch = 0; ch < nchunks; ++ch, ++use) {
        uint4 zq[KCH / 8];
#pragma unroll
        for (int i = 0; i < KCH / 8; ++i) {
          zq[i] = znext[i];
          const bool in_h = ch + 1 < nchunks && key0 + (ch + 1) * KCH + i * 8 < P.h;
          znext[i] = valid && in_h ? __ldg(reinterpret_cast<const uint4*>(zrow + (ch + 1) * KCH + i * 8))
                                   : make_uint4(0, 0, 0, 0);
        }
        // The MMA thread releases a stage tile by tile (128 knot rows each); with the words per key
        // known at compile time (HLC) a tile is waited for just before the first key that touches it,
        // so this stage's first keys are written while the MMAs still read the later tiles of the
        // previous use.  Otherwise all tiles are waited for first.
        if (!HLC && use > 0)
          for (int m = 0; m < P.mtiles; ++m) mbar_wait(pempty + pg * 3 + m, (uint32_t)(use - 1) & 1u, wc);
        const int keys_left = P.h - (key0 + ch * KCH);         // keys of this chunk that exist
#pragma unroll
        for (int q = 0; q < KCH; ++q) {
          if (HLC && use > 0) {
            // tiles touched by words q * HLC .. (q + 1) * HLC - 1 (word w lies in tile w >> 6) that no
            // earlier key touched
            const int t_lo = q == 0 ? 0 : (((q * HLC - 1) >> 6) + 1), t_hi = ((q + 1) * HLC - 1) >> 6;
#pragma unroll
            for (int m = 0; m < 3; ++m)
              if (m >= t_lo && m <= t_hi) mbar_wait(pempty + pg * 3 + m, (uint32_t)(use - 1) & 1u, wc);
          }
          if (have_saved) {
            sts32(row + (saved[q] & 0xffffu) * 4u, 0u);
            sts32(row + (saved[q] >> 16) * 4u, 0u);
          }
          if (valid) {
            const uint4& zc = zq[q >> 3];
            const uint32_t zw[4] = {zc.x, zc.y, zc.z, zc.w};
            const int qq = q & 7;
            const float zz = (qq & 1) ? bf_hi(zw[qq >> 1]) : bf_lo(zw[qq >> 1]);
            uint32_t x0, x1, wo0, wo1;
            phi_pair(zz, P.g, (uint32_t)q * halfL, x0, x1, wo0, wo1);
            if (q >= keys_left) { x0 = 0u; x1 = 0u; }
            sts32(row + wo0 * 4u, x0);
            sts32(row + wo1 * 4u, x1);
            saved[q] = wo0 | (wo1 << 16);
          }
        }
        have_saved = valid;
        fence_async_smem();
        mbar_arrive_warp(pfull + pg);
      }
    }
    // ---- epilogue: accumulators -> float32 partial of this token split
    mbar_wait(done, 0, wc);
    tc_fence_after();
    const int lane_row = (warp & 3) * 32 + lane;
    float* part = P.part + (size_t)blockIdx.y * P.h * L * r;
    for (int ch = pg; ch < nchunks; ch += 2) {
      for (int mt = 0; mt < P.mtiles; ++mt) {
        const int rr = mt * 128 + lane_row;                        // padded knot row within the chunk
        const int kl = rr / LR, bb = rr - kl * LR;
        const int key = key0 + ch * KCH + kl;
        const bool ok = rr < rows && key < P.h && bb < L;           // the pad row of an odd L is dropped
        float* dst = part + ((size_t)key * L + bb) * r;
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((ch * P.mtiles + mt) * r);
        for (int c0 = 0; c0 < r; c0 += 16) {
          float v[16];
          tmem_ld16(taddr + c0, v);
          if (ok) {
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              *reinterpret_cast<float4*>(dst + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          }
        }
      }
    }
    tc_fence_before();
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc(0, 0, 1, 1, 128, r);
      const uint32_t ab_hi = desc_hi(2048u);
      int guse[2] = {0, 0}, puse[2] = {0, 0};
      bool drain = false;
      for (int tp = 0; tp < ntiles; tp += 2) {
        const int npg = min(2, ntiles - tp);
        for (int pg = 0; pg < npg; ++pg)
          drain = mbar_wait(gfull + pg, (uint32_t)guse[pg] & 1u, wc) || drain;
        if (drain) break;
        for (int ch = 0; ch < nchunks; ++ch) {
          for (int pg = 0; pg < npg; ++pg) {
            drain = mbar_wait(pfull + pg, (uint32_t)puse[pg] & 1u, wc);
            ++puse[pg];
            if (drain) break;                        // draining: issue nothing more
            tc_fence_after();
            const uint32_t a_addr = smem_u32(phi_base + (size_t)pg * phi_bytes);
            const uint32_t b_addr = smem_u32(g_base + (size_t)pg * g_bytes);
            const uint32_t first = (tp == 0 && pg == 0) ? 0u : 1u;
            const uint32_t b_lo0 = desc_lo(b_addr, 128u);
            for (int mt = 0; mt < P.mtiles; ++mt) {
              uint32_t a_lo = desc_lo(a_addr + (uint32_t)mt * 16u * 2048u, 128u);
              uint32_t b_lo = b_lo0;
              const uint32_t d_addr = tmem_base + (uint32_t)((ch * P.mtiles + mt) * r);
              umma_f16_split(d_addr, a_lo, ab_hi, b_lo, ab_hi, idesc, first);
#pragma unroll
              for (int ks = 1; ks < 8; ++ks) {
                a_lo += 256u >> 4;
                b_lo += 256u >> 4;
                umma_f16_split(d_addr, a_lo, ab_hi, b_lo, ab_hi, idesc, 1u);
              }
              umma_commit(pempty + pg * 3 + mt);
            }
          }
          if (drain) break;
        }
        if (drain) break;
        for (int pg = 0; pg < npg; ++pg) { umma_commit(gempty + pg); ++guse[pg]; }
      }
      umma_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ gradient-tile loader
    if (lane == 0) {
      int guse[2] = {0, 0};
      for (int ti = 0; ti < ntiles; ++ti) {
        const int pg = ti & 1;
        if (guse[pg] > 0)
          mbar_wait(gempty + pg, (uint32_t)(guse[pg] - 1) & 1u, wc);
        if (*abort_flag) break;
        mbar_arrive_expect_tx(gfull + pg, g_bytes);
        bulk_g2s(g_base + (size_t)pg * g_bytes,
                 reinterpret_cast<const uint8_t*>(P.gimg) + (size_t)(tile_begin + ti) * g_bytes, g_bytes, gfull + pg);
        ++guse[pg];
      }
      if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
  }
  __syncthreads();
  if (warp == 8) {
    mbar_wait_drain(done, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, tmem_cols);
  }
}

__global__ void tc_dc_reduce_kernel(const float* __restrict__ part, int splits, size_t elems, float lambda,
                                    const uint32_t* __restrict__ amax_bits, float* __restrict__ dC,
                                    __nv_bfloat16* __restrict__ dC_cast) {
  float gscale, ginv;
  pow2_scales(*amax_bits, gscale, ginv);
  const float f = lambda * ginv;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += (size_t)gridDim.x * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += part[(size_t)k * elems + i];
    s *= f;
    if (dC) dC[i] = s;
    if (dC_cast) dC_cast[i] = __float2bfloat16_rn(s);
  }
}

// =================================================================================================
// fused backward: dz and dC in one CTA
// =================================================================================================
// A CTA owns a slab of 16 keys and a range of 128-token tiles; tile i belongs to token group i % 2.
// The dz kernel is bound by instruction issue and the dC kernel by shared-memory bandwidth (its
// producers wait half the time for the MMAs that read their stage); run as separate warps of one
// CTA the two fill each other's gaps, and the g tile in shared memory serves both.
//
//   warps 0..7    dz role, groups 0 and 1 (thread = token): the S columns of 4 keys at a time
//                 (S = g T^T, in one of the group's two tensor-memory blocks, so that the next
//                 block is computed while this one is read) -> dz, as tc_dz_kernel does
//   warps 8..15   Phi role, groups 0 and 1: a group fills stages of 64 tokens x 16 keys (two
//                 threads per token, 8 keys each): knot interval and weights -> the two non-zero
//                 words of each key's Phi^T segment, scattered into the stage (A operand of the dC
//                 MMAs); two stages per group, so that one is filled while the other is read
//   warp 16       lane 0 issues the S MMAs of both groups (whichever is ready first)
//   warp 17       lane 0 issues the dC MMAs of both groups (3 M-tiles x 4 K-steps per stage)
//   warp 18       lane 0 loads the slab's transformed table once and streams the g tiles (3-deep ring)
//
// Registers are re-balanced between the roles with setmaxnreg (the kernel starts every warp with
// the same count): the helper warps give registers up, the dz warps take them.
//
// Tensor memory: [group 0: S block 0, S block 1 | group 1: ... | dC accumulators of the slab]
// = 4 * 4*LP + mtiles*r columns.
// Shared memory: four Phi^T stages of 16*L knot rows x 64 tokens, the g ring, the table slab.  A
// stage holds exactly 16*L rows; the MMAs of its last M-tile read up to the next multiple of 128
// rows, i.e. into whatever follows the stage.  Each accumulator row depends on its own A row only
// and the rows past 16*L are never stored, so those reads are harmless.
struct BfParams {
  const __nv_bfloat16* z;
  int64_t zs;
  const __nv_bfloat16* g_act;
  int64_t gas;
  __nv_bfloat16* dz;
  int64_t dzs;
  const __half* gimg;
  const __half* timg;
  const uint32_t* amax_bits;
  float* part;               // [splits][h*L][r]
  int64_t N;
  int h, L, r;
  GridParams g;
  int act;
  float coef;                // lambda * scale
  int mtiles;                // 128-row MMA tiles over the slab's 16*L knot rows
  int dz_f32;                // dz is float32 [N][dzs] instead of bf16
  int roles;                 // bit 0: the dz role runs, bit 1: the Phi role and the dC MMAs run
  int64_t tiles_per_split, tiles_total;
  int32_t* status;
  long long wait_cycles;
};

constexpr int kSlabKeys = 16;
constexpr int kGRing = 3;
constexpr int kBfThreads = 640;
constexpr int kAux0 = 16;                      // first helper warp
// register counts per role (multiples of 8); 256 * kRegsDz + 256 * kRegsPhi + 128 * kRegsAux must
// not exceed kBfThreads * the count the kernel is compiled for (96)
constexpr int kRegsDz = 128, kRegsPhi = 88, kRegsAux = 40;
#ifndef SKV_POLL_NS
#define SKV_POLL_NS 20
#endif
constexpr unsigned kPollNs = SKV_POLL_NS;               // pause of an MMA issuer that found nothing ready

template <int R> __device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}
template <int R> __device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}

template <int LB, int NC, bool RELU>
__global__ void __launch_bounds__(kBfThreads, 1) tc_bwd_fused_kernel(const BfParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int L = P.L, r = P.r;
  constexpr int LP = 8 * LB;
  constexpr uint32_t bcols = (uint32_t)(4 * LP);                    // columns of one S block (4 keys)
  const uint32_t phi_bytes = (uint32_t)((kSlabKeys * L + 7) / 8) * 1024u;   // one 64-token stage
  const uint32_t g_bytes = (uint32_t)(128 * r * 2);
  const uint32_t t_bytes = (uint32_t)(kChunkKeys * LP * r * 2);     // table image of 8 keys
  uint8_t* phi_base = smem;                                          // [2 groups][2][phi_bytes]
  uint8_t* g_base = phi_base + 4 * (size_t)phi_bytes;                // [kGRing][g_bytes]
  uint8_t* t_base = g_base + (size_t)kGRing * g_bytes;               // [2][t_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(t_base + 2 * (size_t)t_bytes);
  uint64_t* gfull = bars;                  // [kGRing] loader -> MMA issuers
  uint64_t* gempty = gfull + kGRing;       // [kGRing] both MMA issuers -> loader (2 arrivals)
  uint64_t* tfull = gempty + kGRing;       // [1]
  uint64_t* sfull = tfull + 1;             // [2 groups][2] S issuer -> dz group
  uint64_t* sempty = sfull + 4;            // [2 groups][2] dz group -> S issuer
  uint64_t* pfull = sempty + 4;            // [2 groups][2] Phi group -> dC issuer
  uint64_t* pempty = pfull + 4;            // [2 groups][2] dC issuer -> Phi group
  uint64_t* done = pempty + 4;             // [2] all MMAs of the S issuer / the dC issuer complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutBwd, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int key0 = blockIdx.x * kSlabKeys;
  const int64_t tile_begin = (int64_t)blockIdx.y * P.tiles_per_split;
  const int ntiles = (int)min(P.tiles_per_split, P.tiles_total - tile_begin);
  const uint32_t dcol0 = 4u * bcols;
  uint32_t tmem_cols = 32;
  while (tmem_cols < dcol0 + (uint32_t)(P.mtiles * r)) tmem_cols <<= 1;

  if (tid == 0) {
    const uint32_t issuers = (uint32_t)((P.roles & 1) + ((P.roles >> 1) & 1));
    for (int i = 0; i < kGRing; ++i) { mbar_init(gfull + i, 1); mbar_init(gempty + i, issuers); }
    mbar_init(tfull, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(sfull + i, 1);
      mbar_init(sempty + i, 4);
      mbar_init(pfull + i, 4);
      mbar_init(pempty + i, 1);
    }
    mbar_init(done + 0, 1);
    mbar_init(done + 1, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  {
    uint4* p = reinterpret_cast<uint4*>(phi_base);
    const uint32_t n16 = 4 * phi_bytes / 16;
    for (uint32_t i = tid; i < n16; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == kAux0) tmem_alloc(tmem_slot, tmem_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 8) {
    // ------------------------------------------------------------------ dz role
    reg_inc<kRegsDz>();
    const int pg = warp >> 2;
    const int t = tid & 127;
    const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)pg * 2u * bcols;
    float gscale, ginv;
    pow2_scales(*P.amax_bits, gscale, ginv);
    float cscale, cinv;
    pow2_scales(P.amax_bits[kAmaxC], cscale, cinv);
    const float coef = P.coef * ginv * cinv;
    const int act = P.act;
    const bool has_ga = P.g_act != nullptr;
    auto load_rows = [&](int ti, uint4 (&zv)[2], uint4 (&gv)[2], bool& valid, __nv_bfloat16*& dzrow) {
      const int64_t n = (tile_begin + ti) * 128 + t;
      valid = ti < ntiles && n < P.N;
      const int64_t nn = valid ? n : 0;
      const __nv_bfloat16* zrow = P.z + nn * P.zs + key0;
      const __nv_bfloat16* garow = has_ga ? P.g_act + nn * P.gas + key0 : nullptr;
      dzrow = P.dz + nn * P.dzs + key0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        zv[i] = valid ? __ldg(reinterpret_cast<const uint4*>(zrow + i * 8)) : make_uint4(0, 0, 0, 0);
        gv[i] = valid && has_ga ? __ldg(reinterpret_cast<const uint4*>(garow + i * 8)) : make_uint4(0, 0, 0, 0);
      }
    };
    uint4 znext[2], ganext[2];
    bool vnext;
    __nv_bfloat16* dznext;
    load_rows(pg, znext, ganext, vnext, dznext);
    int use = 0;                                     // S blocks this group has consumed
    for (int ti = pg; ti < ntiles && (P.roles & 1); ti += 2) {
      const uint4 zq[2] = {znext[0], znext[1]}, gaq[2] = {ganext[0], ganext[1]};
      const bool valid = vnext;
      __nv_bfloat16* dzrow = dznext;
      load_rows(ti + 2, znext, ganext, vnext, dznext);   // the group's next tile: request its rows now
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {               // 8 keys per pass: two S blocks of 4 keys, unrolled
        const uint4 zc = hf ? zq[1] : zq[0], gc = hf ? gaq[1] : gaq[0];
        const uint32_t zw[4] = {zc.x, zc.y, zc.z, zc.w};
        const uint32_t gw[4] = {gc.x, gc.y, gc.z, gc.w};
        float outv[kChunkKeys];
#pragma unroll
        for (int qt = 0; qt < 2; ++qt, ++use) {
          const uint32_t blk = trow + (uint32_t)(use & 1) * bcols;
          uint32_t bufa[LB][8], bufb[LB][8];
          mbar_wait(sfull + pg * 2 + (use & 1), (uint32_t)(use >> 1) & 1u, wc);
          tc_fence_after();
          tmem_ld_key<LB, NC>(blk, bufa);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int q = qt * 4 + q4;
            if (q4 & 1) tmem_wait_key<LB, NC>(bufb); else tmem_wait_key<LB, NC>(bufa);
            if (q4 + 1 < 4) {
              if (q4 & 1) tmem_ld_key<LB, NC>(blk + (uint32_t)((q4 + 1) * LP), bufa);
              else tmem_ld_key<LB, NC>(blk + (uint32_t)((q4 + 1) * LP), bufb);
            }
            const float zz = (q & 1) ? bf_hi(zw[q >> 1]) : bf_lo(zw[q >> 1]);
            const float u = __fmaf_rn(__fsub_rn(zz, P.g.lo), P.g.scale, 0.0f);
            const bool active = __float_as_uint(u) <= __float_as_uint(P.g.Gm1f);
            const float uc = fminf(fmaxf(u, 0.0f), P.g.Gm1f);
            const float acc = (q4 & 1) ? dz_key_sum<LB, NC>(bufb, uc) : dz_key_sum<LB, NC>(bufa, uc);
            float o = active ? coef * acc : 0.0f;
            if (has_ga) {
              const float ga = (q & 1) ? bf_hi(gw[q >> 1]) : bf_lo(gw[q >> 1]);
              const float dphi = RELU ? 2.0f * fmaxf(zz, 0.0f) : act_grad(zz, act);
              o = fmaf(ga, dphi, o);
            }
            outv[q] = o;
          }
          tc_fence_before();
          mbar_arrive_warp(sempty + pg * 2 + (use & 1));
        }
        if (valid) {
          if (P.dz_f32) {
            float* o = reinterpret_cast<float*>(P.dz) + (dzrow - P.dz) + hf * 8;
            *reinterpret_cast<float4*>(o) = make_float4(outv[0], outv[1], outv[2], outv[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(outv[4], outv[5], outv[6], outv[7]);
          } else {
            *reinterpret_cast<uint4*>(dzrow + hf * 8) =
                make_uint4(pack_bf2(outv[0], outv[1]), pack_bf2(outv[2], outv[3]), pack_bf2(outv[4], outv[5]),
                           pack_bf2(outv[6], outv[7]));
          }
        }
      }
    }
    // ---- epilogue: the slab's accumulators -> float32 partial of this token split
    if (P.roles & 2) mbar_wait(done + 1, 0, wc);
    tc_fence_after();
    const int lane_row = (warp & 3) * 32 + lane;
    const int rows = kSlabKeys * L;
    float* part = P.part + ((size_t)blockIdx.y * P.h + key0) * L * r;
    for (int mt = pg; mt < P.mtiles && (P.roles & 2); mt += 2) {
      const int rr = mt * 128 + lane_row;
      const bool ok = rr < rows;
      float* dst = part + (size_t)rr * r;
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + dcol0 + (uint32_t)(mt * r);
      for (int c0 = 0; c0 < r; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + c0, v);
        if (ok) {
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4*>(dst + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
      }
    }
    tc_fence_before();
  } else if (warp < kAux0) {
    // ------------------------------------------------------------------ Phi role
    reg_dec<kRegsPhi>();
    const int pg = (warp - 8) >> 2;
    const int t = tid & 127;
    const int tok = t & 63, kh = t >> 6;             // token of the half tile, key half of the slab
    const uint32_t t_off = (uint32_t)(tok & 7) * 16u + (uint32_t)(tok >> 3) * 128u;
    const uint32_t row0 = smem_u32(phi_base + (size_t)(pg * 2) * phi_bytes) + t_off;
    const uint32_t halfL = (uint32_t)L >> 1;
    // first word index (< 16 * L / 2 <= 255) of the pair each key wrote, per stage: 8 keys x 8 bits
    // in two registers; the positions are cleared before the stage is filled again
    uint32_t sav[2][2] = {{0u, 0u}, {0u, 0u}};
    // fill f of this group: tile pg + 2 * (f / 2), token half f % 2, stage f % 2
    const int nfill = 2 * ((ntiles - pg + 1) / 2);
    auto load_z = [&](int f, uint4& zv, bool& valid) {
      const int ti = pg + 2 * (f >> 1);
      const int64_t n = (tile_begin + ti) * 128 + (f & 1) * 64 + tok;
      valid = f < nfill && n < P.N;
      zv = valid ? __ldg(reinterpret_cast<const uint4*>(P.z + n * P.zs + key0 + kh * 8)) : make_uint4(0, 0, 0, 0);
    };
    uint4 znext;
    bool vnext;
    load_z(0, znext, vnext);
#pragma unroll 1
    for (int f = 0; f < nfill && (P.roles & 2); ++f) {
      const int st = f & 1;
      const uint4 zc = znext;
      const bool valid = vnext;
      load_z(f + 1, znext, vnext);                   // the next fill's rows are requested now
      const uint32_t row = row0 + (uint32_t)st * phi_bytes;
      // the stage is free once the dC MMAs of its previous fill are done
      if (f > 1) mbar_wait(pempty + pg * 2 + st, (uint32_t)((f >> 1) - 1) & 1u, wc);
#pragma unroll 1
      for (int i = 0; i < 2; ++i) {                  // 4 keys per pass (small body, see the dz role)
        const uint32_t zw[2] = {i ? zc.z : zc.x, i ? zc.w : zc.y};
        const uint32_t old = st ? (i ? sav[1][1] : sav[1][0]) : (i ? sav[0][1] : sav[0][0]);
        uint32_t now = 0u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (f > 1) {
            const uint32_t c0 = (old >> (8 * q)) & 0xffu, c1 = c0 + 1u;
            sts32(row + (c0 + (c0 >> 2) * 252u) * 4u, 0u);
            sts32(row + (c1 + (c1 >> 2) * 252u) * 4u, 0u);
          }
          const float zz = (q & 1) ? bf_hi(zw[q >> 1]) : bf_lo(zw[q >> 1]);
          uint32_t x0, x1, s0;
          phi_pair_s(zz, P.g, (uint32_t)(kh * 8 + i * 4 + q) * halfL, x0, x1, s0);
          if (!valid) { x0 = 0u; x1 = 0u; }
          const uint32_t s1 = s0 + 1u;
          sts32(row + (s0 + (s0 >> 2) * 252u) * 4u, x0);
          sts32(row + (s1 + (s1 >> 2) * 252u) * 4u, x1);
          now |= s0 << (8 * q);
        }
        if (st) { if (i) sav[1][1] = now; else sav[1][0] = now; }
        else { if (i) sav[0][1] = now; else sav[0][0] = now; }
      }
      fence_async_smem();
      mbar_arrive_warp(pfull + pg * 2 + st);
    }
  } else {
    reg_dec<kRegsAux>();
    if (warp == kAux0) {
      // ---------------------------------------------------------------- S MMAs (both groups)
      if (lane == 0 && (P.roles & 1)) {
        mbar_wait(tfull, 0, wc);
        const uint32_t rb = (uint32_t)(r / 8) * 128u;
        const uint32_t a_hi = desc_hi(128u), b_hi = desc_hi(rb);
        const uint32_t idesc = instr_desc(0, 0, 0, 0, 128, (int)bcols);
        // whichever group is ready first is served (the groups drift apart; serving them in a fixed
        // order would tie each to the slower one)
        int it[2] = {0, 0};
        const int total[2] = {4 * ((ntiles + 1) / 2), 4 * (ntiles / 2)};
        long long t_last = clock64();
        while ((it[0] < total[0] || it[1] < total[1]) && !*abort_flag) {
          bool progressed = false;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            if (it[pg] >= total[pg]) continue;
            const int k = it[pg], ti = pg + 2 * (k >> 2), qt = k & 3, sb = k & 1, b = ti % kGRing;
            if (qt == 0 && !mbar_test_wait(gfull + b, (uint32_t)(ti / kGRing) & 1u)) continue;
            if (k > 1 && !mbar_test_wait(sempty + pg * 2 + sb, (uint32_t)((k >> 1) - 1) & 1u)) continue;
            tc_fence_after();
            uint32_t a_lo = desc_lo(smem_u32(g_base + (size_t)b * g_bytes), 2048u);
            uint32_t b_lo = desc_lo(smem_u32(t_base) + (uint32_t)qt * (uint32_t)(LP / 2) * rb, 128u);
            const uint32_t d_addr = tmem_base + (uint32_t)(pg * 2 + sb) * bcols;
            for (int ks = 0; ks < r / 16; ++ks) {
              umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, ks > 0 ? 1u : 0u);
              a_lo += 4096u >> 4;
              b_lo += 256u >> 4;
            }
            umma_commit(sfull + pg * 2 + sb);
            if (qt == 3) umma_commit(gempty + b);        // this issuer is done with the g tile
            ++it[pg];
            progressed = true;
          }
          if (progressed) t_last = clock64();
          else if (clock64() - t_last > P.wait_cycles) wait_give_up(wc);
          else __nanosleep(kPollNs);
        }
        umma_commit(done + 0);
      }
    } else if (warp == kAux0 + 1) {
      // ---------------------------------------------------------------- dC MMAs (both groups)
      if (lane == 0 && (P.roles & 2)) {
        const uint32_t idesc = instr_desc(0, 0, 1, 1, 128, r);
        const uint32_t a_hi = desc_hi(1024u), b_hi = desc_hi(2048u);
        int it[2] = {0, 0};
        const int total[2] = {2 * ((ntiles + 1) / 2), 2 * (ntiles / 2)};
        bool first = true;
        long long t_last = clock64();
        while ((it[0] < total[0] || it[1] < total[1]) && !*abort_flag) {
          bool progressed = false;
#pragma unroll
          for (int pg = 0; pg < 2; ++pg) {
            if (it[pg] >= total[pg]) continue;
            const int f = it[pg], ti = pg + 2 * (f >> 1), st = f & 1, b = ti % kGRing;
            if (!mbar_test_wait(pfull + pg * 2 + st, (uint32_t)(f >> 1) & 1u)) continue;
            if (!mbar_test_wait(gfull + b, (uint32_t)(ti / kGRing) & 1u)) continue;
            tc_fence_after();
            const uint32_t a_addr = smem_u32(phi_base + (size_t)(pg * 2 + st) * phi_bytes);
            // tokens 64 * st .. of the g tile: token groups 8 * st ..
            const uint32_t b_lo0 = desc_lo(smem_u32(g_base + (size_t)b * g_bytes) + (uint32_t)st * 8u * 128u, 128u);
            for (int mt = 0; mt < P.mtiles; ++mt) {
              uint32_t a_lo = desc_lo(a_addr + (uint32_t)mt * 16u * 1024u, 128u);
              uint32_t b_lo = b_lo0;
              const uint32_t d_addr = tmem_base + dcol0 + (uint32_t)(mt * r);
              umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, first ? 0u : 1u);
#pragma unroll
              for (int ks = 1; ks < 4; ++ks) {
                a_lo += 256u >> 4;
                b_lo += 256u >> 4;
                umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, 1u);
              }
            }
            first = false;
            umma_commit(pempty + pg * 2 + st);
            if (st == 1) umma_commit(gempty + b);
            ++it[pg];
            progressed = true;
          }
          if (progressed) t_last = clock64();
          else if (clock64() - t_last > P.wait_cycles) wait_give_up(wc);
          else __nanosleep(kPollNs);
        }
        umma_commit(done + 1);
      }
    } else if (warp == kAux0 + 2) {
      // ---------------------------------------------------------------- loader
      if (lane == 0) {
        mbar_arrive_expect_tx(tfull, 2 * t_bytes);
        bulk_g2s(t_base, reinterpret_cast<const uint8_t*>(P.timg) + (size_t)(key0 / kChunkKeys) * t_bytes,
                 2 * t_bytes, tfull);
        for (int ti = 0; ti < ntiles; ++ti) {
          const int b = ti % kGRing;
          if (ti >= kGRing) mbar_wait(gempty + b, (uint32_t)((ti / kGRing) - 1) & 1u, wc);
          if (*abort_flag) break;
          mbar_arrive_expect_tx(gfull + b, g_bytes);
          bulk_g2s(g_base + (size_t)b * g_bytes,
                   reinterpret_cast<const uint8_t*>(P.gimg) + (size_t)(tile_begin + ti) * g_bytes, g_bytes, gfull + b);
        }
        if (*abort_flag) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000) {}
        }
      }
    }
  }
  __syncthreads();
  if (warp == kAux0) {
    if (P.roles & 1) mbar_wait_drain(done + 0, 0, P.wait_cycles);
    if (P.roles & 2) mbar_wait_drain(done + 1, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------------------------------------
struct DzPlan { int groups, lb, splits, chunks_per_split, tstages; size_t smem; };

bool plan_dz(const skv_problem& p, DzPlan* o) {
  const int lb = (p.L - 1 + 7) / 8;                  // 8-column blocks per key; columns L-1.. are padding
  if (lb < 1 || lb > 6) return false;
  const int ncols = kChunkKeys * 8 * lb;
  const int groups = 2 * ncols <= 512 ? 2 : 1;
  o->groups = groups;
  o->lb = lb;
  int tstages = kTStages;
  auto smem_for = [&](int ts) { return (size_t)groups * 128 * p.r * 2 + (size_t)ts * kChunkKeys * 8 * lb * p.r * 2 + 256; };
  while (tstages > 2 && smem_for(tstages) > kSmemMax) --tstages;
  o->tstages = tstages;
  o->smem = smem_for(tstages);
  if (o->smem > kSmemMax) return false;
  const int chunks = p.h / kChunkKeys;
  const int64_t tiles = (p.N + 128 * groups - 1) / (128 * groups);
  int best = 1;
  double best_eff = 0.0;
  const int max_splits = chunks >= 16 ? (chunks / 8 < 16 ? chunks / 8 : 16) : 1;
  for (int ks = 1; ks <= max_splits; ++ks) {
    const double waves = (double)(tiles > 0 ? tiles : 1) * ks / kPlanSMs;
    const double eff = waves / (double)(int64_t)(waves + 0.999999);
    if (eff > best_eff + 0.04) { best_eff = eff; best = ks; }
  }
  o->chunks_per_split = (chunks + best - 1) / best;
  o->splits = (chunks + o->chunks_per_split - 1) / o->chunks_per_split;
  return true;
}

struct DcPlan { int kch, mtiles, slab_chunks, slabs, splits; int64_t tiles_total, tiles_per_split; size_t smem; };

bool plan_dc(const skv_problem& p, DcPlan* o) {
  const int LR = (p.L + 1) & ~1;
  for (int kch = 16; kch >= 8; kch /= 2) {
    const int rows = kch * LR;
    const int mtiles = (rows + 127) / 128;
    if (mtiles > 3) continue;
    const size_t smem = 2 * (size_t)mtiles * 16 * 2048 + 2 * (size_t)128 * p.r * 2 + 256;
    if (smem > kSmemMax) continue;
    int slab_chunks = 512 / (mtiles * p.r);
    if (slab_chunks < 1) continue;
    if (slab_chunks > 8) slab_chunks = 8;
    const int chunks = (p.h + kch - 1) / kch;
    if (slab_chunks > chunks) slab_chunks = chunks;
    o->kch = kch;
    o->mtiles = mtiles;
    o->slab_chunks = slab_chunks;
    o->slabs = (chunks + slab_chunks - 1) / slab_chunks;
    o->smem = smem;
    o->tiles_total = (p.N + 127) / 128;
    const int64_t tt = o->tiles_total > 0 ? o->tiles_total : 1;
    int best = 1;
    double best_eff = 0.0;
    const int64_t max_splits = tt / 4 < 1 ? 1 : (tt / 4 > 32 ? 32 : tt / 4);
    for (int ns = 1; ns <= max_splits; ++ns) {
      const double waves = (double)o->slabs * ns / kPlanSMs;
      const double eff = waves / (double)(int64_t)(waves + 0.999999);
      if (eff > best_eff + 0.04) { best_eff = eff; best = ns; }
    }
    o->tiles_per_split = (tt + best - 1) / best;
    o->splits = (int)((tt + o->tiles_per_split - 1) / o->tiles_per_split);
    return true;
  }
  return false;
}

struct FusedPlan { int lb, mtiles, slabs, splits; int64_t tiles_total, tiles_per_split; size_t smem; };

// The fused kernel covers shapes whose slab fits: even L up to 24 (16 keys x L rows in three M-tiles),
// r small enough for the tensor-memory plan, h a multiple of the slab.
bool plan_fused(const skv_problem& p, FusedPlan* o) {
  if (p.L % 2 || p.L > 24 || p.h % kSlabKeys || p.N < 1) return false;
  const int lb = (p.L - 1 + 7) / 8;
  if (lb < 1 || lb > 3) return false;
  const int mtiles = (kSlabKeys * p.L + 127) / 128;
  if (2 * kChunkKeys * 8 * lb + mtiles * p.r > 512) return false;
  const size_t phi_bytes = (size_t)((kSlabKeys * p.L + 7) / 8) * 1024;      // one 64-token stage
  const size_t smem = 4 * phi_bytes + (size_t)kGRing * 128 * p.r * 2 + 2 * (size_t)kChunkKeys * 8 * lb * p.r * 2 + 256;
  if (smem > kSmemMax) return false;
  // the last M-tile of the last stage reads past the stage: that read must stay inside the allocation
  if (3 * phi_bytes + (size_t)mtiles * 16 * 1024 > smem) return false;
  o->lb = lb;
  o->mtiles = mtiles;
  o->slabs = p.h / kSlabKeys;
  o->smem = smem;
  o->tiles_total = (p.N + 127) / 128;
  const int64_t tt = o->tiles_total;
  int best = 1;
  double best_eff = 0.0;
  const int64_t max_splits = tt / 4 < 1 ? 1 : (tt / 4 > 32 ? 32 : tt / 4);
  for (int ns = 1; ns <= max_splits; ++ns) {
    const double waves = (double)o->slabs * ns / kPlanSMs;
    const double eff = waves / (double)(int64_t)(waves + 0.999999);
    if (eff > best_eff + 0.04) { best_eff = eff; best = ns; }
  }
  o->tiles_per_split = (tt + best - 1) / best;
  o->splits = (int)((tt + o->tiles_per_split - 1) / o->tiles_per_split);
  return true;
}

size_t timg_bytes(const skv_problem& p) {
  const int lb = (p.L - 1 + 7) / 8;
  return align256((size_t)p.h * 8 * lb * p.r * sizeof(__half));
}

size_t gimg_bytes(const skv_problem& p) {
  const int64_t tiles = ((p.N + 255) / 256) * 2;
  return align256((size_t)(tiles > 0 ? tiles : 2) * 128 * p.r * 2);
}

}  // namespace

bool bwd_eligible(const skv_problem& p) {
  if (!fwd_eligible(p)) return false;
  DzPlan a;
  DcPlan b;
  return plan_dz(p, &a) && plan_dc(p, &b);
}

size_t bwd_scratch_bytes(const skv_problem& p) {
  DcPlan d;
  if (!plan_dc(p, &d)) return 0;
  int splits = d.splits;
  FusedPlan f;
  if (plan_fused(p, &f) && f.splits > splits) splits = f.splits;     // whichever path a call takes fits
  return 256 + gimg_bytes(p) + timg_bytes(p) + align256((size_t)splits * p.h * p.L * p.r * sizeof(float));
}

int backward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, const void* g_act, int64_t gas,
             const void* g_delta, int64_t gds, void* dz, int64_t dzs, float* dC, void* dC_cast, void* scratch,
             size_t scratch_bytes) {
  const skv_problem& p = c.p;
  DzPlan zp;
  DcPlan dp;
  if (!plan_dz(p, &zp) || !plan_dc(p, &dp)) return SKV_ERR_UNSUPPORTED;
  if (scratch_bytes < bwd_scratch_bytes(p)) return SKV_ERR_SCRATCH;
  uint8_t* base = reinterpret_cast<uint8_t*>(scratch);
  uint32_t* amax = reinterpret_cast<uint32_t*>(base);
  __half* gimg = reinterpret_cast<__half*>(base + 256);
  __half* timg = reinterpret_cast<__half*>(base + 256 + gimg_bytes(p));
  float* part = reinterpret_cast<float*>(base + 256 + gimg_bytes(p) + timg_bytes(p));

  if (cudaMemsetAsync(amax, 0, 256, c.stream) != cudaSuccess) return SKV_ERR_LAUNCH;
  {
    const int64_t total = p.N * p.r;
    const unsigned grid = (unsigned)((total + 2047) / 2048 < 296 ? (total + 2047) / 2048 : 296);
    tc_amax_kernel<<<grid, 256, 0, c.stream>>>((const __nv_bfloat16*)g_delta, gds, p.N, p.r, amax + kAmaxG);
    if (dz) {
      const int64_t crows = (int64_t)p.h * p.L;
      const unsigned cgrid = (unsigned)((crows * p.r + 2047) / 2048 < 296 ? (crows * p.r + 2047) / 2048 : 296);
      tc_amax_kernel<<<cgrid, 256, 0, c.stream>>>((const __nv_bfloat16*)C, p.r, crows, p.r, amax + kAmaxC);
      note_launches(1);
    }
    const int64_t tiles = ((p.N + 255) / 256) * 2;
    const int64_t pieces = tiles * 128 * (p.r / 8);
    const unsigned pgrid = (unsigned)((pieces + 255) / 256 < 2368 ? (pieces + 255) / 256 : 2368);
    tc_pack_g_kernel<<<pgrid, 256, 0, c.stream>>>((const __nv_bfloat16*)g_delta, gds, p.N, p.r, tiles, amax, gimg);
    note_launches(2);
    if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
  }

  FusedPlan fp;
  if (fused_backward_roles() && dz && (dC || dC_cast) && plan_fused(p, &fp)) {
    const size_t pieces = (size_t)p.h * 8 * fp.lb * (p.r / 8);
    const unsigned tgrid = (unsigned)((pieces + 255) / 256 < 2048 ? (pieces + 255) / 256 : 2048);
    tc_pack_t_kernel<<<tgrid, 256, 0, c.stream>>>((const __nv_bfloat16*)C, timg, p.h, p.L, 8 * fp.lb, p.r, amax);
    note_launches(1);
    BfParams P;
    P.z = (const __nv_bfloat16*)z;
    P.zs = zs;
    P.g_act = (const __nv_bfloat16*)g_act;
    P.gas = gas;
    P.dz = (__nv_bfloat16*)dz;
    P.dzs = dzs;
    P.gimg = gimg;
    P.timg = timg;
    P.amax_bits = amax;
    P.part = part;
    P.N = p.N;
    P.h = p.h;
    P.L = p.L;
    P.r = p.r;
    P.g = c.g;
    P.act = p.activation;
    P.coef = p.lambda_scale * c.g.scale;
    P.mtiles = fp.mtiles;
    P.dz_f32 = p.dz_f32;
    P.roles = fused_backward_roles();
    P.tiles_per_split = fp.tiles_per_split;
    P.tiles_total = fp.tiles_total;
    P.status = c.status;
    P.wait_cycles = wait_cycle_limit();
    dim3 grid((unsigned)fp.slabs, (unsigned)fp.splits);
    cudaError_t err = cudaErrorInvalidValue;
#define SKV_BF_CASE(LB_, NC_, COND_)                                                                               \
  if (err == cudaErrorInvalidValue && fp.lb == LB_ && (COND_)) {                                                   \
    if (p.activation == SKV_ACT_RELU_SQ) {                                                                         \
      err = cudaFuncSetAttribute(tc_bwd_fused_kernel<LB_, NC_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)fp.smem);                                                                    \
      if (err == cudaSuccess) tc_bwd_fused_kernel<LB_, NC_, true><<<grid, kBfThreads, fp.smem, c.stream>>>(P);            \
    } else {                                                                                                       \
      err = cudaFuncSetAttribute(tc_bwd_fused_kernel<LB_, NC_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,\
                                 (int)fp.smem);                                                                    \
      if (err == cudaSuccess) tc_bwd_fused_kernel<LB_, NC_, false><<<grid, kBfThreads, fp.smem, c.stream>>>(P);           \
    }                                                                                                              \
  }
    SKV_BF_CASE(3, 21, p.L == 22) SKV_BF_CASE(2, 15, p.L == 16)
    SKV_BF_CASE(1, 8, true) SKV_BF_CASE(2, 16, true) SKV_BF_CASE(3, 24, true)
#undef SKV_BF_CASE
    note_launches(1);
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) { cudaGetLastError(); return SKV_ERR_LAUNCH; }
    const size_t elems = (size_t)p.h * p.L * p.r;
    const unsigned rgrid = (unsigned)((elems + 255) / 256 < 4096 ? (elems + 255) / 256 : 4096);
    tc_dc_reduce_kernel<<<rgrid, 256, 0, c.stream>>>(part, fp.splits, elems, p.lambda_scale, amax, dC,
                                                     (__nv_bfloat16*)dC_cast);
    note_launches(1);
    return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_LAUNCH;
  }

  if (dz) {
    const size_t pieces = (size_t)p.h * 8 * zp.lb * (p.r / 8);
    const unsigned tgrid = (unsigned)((pieces + 255) / 256 < 2048 ? (pieces + 255) / 256 : 2048);
    tc_pack_t_kernel<<<tgrid, 256, 0, c.stream>>>((const __nv_bfloat16*)C, timg, p.h, p.L, 8 * zp.lb, p.r, amax);
    note_launches(1);
    DzParams P;
    P.z = (const __nv_bfloat16*)z;
    P.zs = zs;
    P.g_act = (const __nv_bfloat16*)g_act;
    P.gas = gas;
    P.dz = (__nv_bfloat16*)dz;
    P.dzs = dzs;
    P.gimg = gimg;
    P.timg = timg;
    P.amax_bits = amax;
    P.N = p.N;
    P.h = p.h;
    P.L = p.L;
    P.r = p.r;
    P.g = c.g;
    P.act = p.activation;
    P.coef = p.lambda_scale * c.g.scale;
    P.chunks_total = p.h / kChunkKeys;
    P.chunks_per_split = zp.chunks_per_split;
    P.tstages = zp.tstages;
    P.dz_f32 = p.dz_f32;
    P.wait_cycles = wait_cycle_limit();
    P.status = c.status;
    const int64_t tiles = (p.N + 128 * zp.groups - 1) / (128 * zp.groups);
    dim3 grid((unsigned)tiles, (unsigned)zp.splits);
    const unsigned threads = 128 * zp.groups + 64;
    cudaError_t err = cudaErrorInvalidValue;
    // NC_ = L - 1 useful columns per key for the knot counts in common use, all 8 * LB_ otherwise
#define SKV_DZ_CASE(G_, LB_, NC_, COND_)                                                                           \
  if (err == cudaErrorInvalidValue && zp.groups == G_ && zp.lb == LB_ && (COND_)) {                                \
    if (p.activation == SKV_ACT_RELU_SQ) {                                                                         \
      err = cudaFuncSetAttribute(tc_dz_kernel<G_, LB_, NC_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 (int)zp.smem);                                                                    \
      if (err == cudaSuccess) tc_dz_kernel<G_, LB_, NC_, true><<<grid, threads, zp.smem, c.stream>>>(P);           \
    } else {                                                                                                       \
      err = cudaFuncSetAttribute(tc_dz_kernel<G_, LB_, NC_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                 (int)zp.smem);                                                                    \
      if (err == cudaSuccess) tc_dz_kernel<G_, LB_, NC_, false><<<grid, threads, zp.smem, c.stream>>>(P);          \
    }                                                                                                              \
  }
    SKV_DZ_CASE(2, 3, 21, p.L == 22) SKV_DZ_CASE(2, 2, 15, p.L == 16) SKV_DZ_CASE(1, 6, 41, p.L == 42)
    SKV_DZ_CASE(2, 1, 8, true) SKV_DZ_CASE(2, 2, 16, true) SKV_DZ_CASE(2, 3, 24, true) SKV_DZ_CASE(2, 4, 32, true)
    SKV_DZ_CASE(1, 5, 40, true) SKV_DZ_CASE(1, 6, 48, true)
#undef SKV_DZ_CASE
    note_launches(1);
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) { cudaGetLastError(); return SKV_ERR_LAUNCH; }
  }

  if (dC || dC_cast) {
    DcParams P;
    P.z = (const __nv_bfloat16*)z;
    P.zs = zs;
    P.gimg = gimg;
    P.part = part;
    P.N = p.N;
    P.h = p.h;
    P.L = p.L;
    P.r = p.r;
    P.g = c.g;
    P.LR = (p.L + 1) & ~1;
    P.kch = dp.kch;
    P.mtiles = dp.mtiles;
    P.slab_chunks = dp.slab_chunks;
    P.tiles_per_split = dp.tiles_per_split;
    P.tiles_total = dp.tiles_total;
    P.status = c.status;
    P.wait_cycles = wait_cycle_limit();
    dim3 grid((unsigned)dp.slabs, (unsigned)dp.splits);
    cudaError_t err;
    if (dp.kch == 16) {
      if (P.LR == 22) {
        err = cudaFuncSetAttribute(tc_dc_kernel<16, 11>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dp.smem);
        if (err == cudaSuccess) tc_dc_kernel<16, 11><<<grid, 320, dp.smem, c.stream>>>(P);
      } else {
        err = cudaFuncSetAttribute(tc_dc_kernel<16, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dp.smem);
        if (err == cudaSuccess) tc_dc_kernel<16, 0><<<grid, 320, dp.smem, c.stream>>>(P);
      }
    } else {
      err = cudaFuncSetAttribute(tc_dc_kernel<8, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dp.smem);
      if (err == cudaSuccess) tc_dc_kernel<8, 0><<<grid, 320, dp.smem, c.stream>>>(P);
    }
    note_launches(1);
    if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) { cudaGetLastError(); return SKV_ERR_LAUNCH; }
    const size_t elems = (size_t)p.h * p.L * p.r;
    const unsigned rgrid = (unsigned)((elems + 255) / 256 < 4096 ? (elems + 255) / 256 : 4096);
    tc_dc_reduce_kernel<<<rgrid, 256, 0, c.stream>>>(part, dp.splits, elems, p.lambda_scale, amax, dC,
                                                     (__nv_bfloat16*)dC_cast);
    note_launches(1);
    if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
  }
  return SKV_OK;
}

}  // namespace tc
}  // namespace skv
