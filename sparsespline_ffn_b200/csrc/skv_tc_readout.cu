// Readout of the feature without materialising it:
//
//   y[N, D] = act(z)[N, h] * W[:, :h]^T  +  (lambda * delta)[N, r] * W[:, h:h+r]^T        (bf16, float32 accumulate)
//
// which is what spline_kv_fwd_fused_cuda of the reference returns
// (src/sparsespline_ffn/cuda_ext/spline_kv_fwd.cu:307-417: activation buffer, delta, two library GEMMs and
// an add).  Here it is one tcgen05 GEMM over the virtual operand [act(z) | lambda*delta] of K = h + r
// columns: the activation is applied to the z tile on its way from global to shared memory, so neither
// act(z) nor the concatenated feature is ever written to HBM; delta (bf16, lambda applied) comes from the
// feature kernel run in its delta-only mode just before.
//
// One persistent CTA per SM walks output tiles of 256 tokens x 256 outputs (two 128-row MMAs share each
// B tile, which halves the L2 traffic per flop of a 128 x 256 tile; all 512 tensor-memory columns hold
// the two accumulators):
//   warp  9    loader (lane 0): per stage one tiled TMA load of the 256 x 64 z (or delta) tile, 128-byte
//              swizzle, zero fill past N and h, and one 32 KB bulk copy from the pre-tiled image of W
//   warps 0-7  ReLU^2 in place on the landed z tile (elementwise, so the swizzled layout does not matter);
//              nothing to do for the identity activation.  After a tile's last stage the same warps are
//              its epilogue (accumulator -> bf16 -> y)
//   warp  8    MMA issue (lane 0): 128 x 256 x 16 per instruction
// Three stages of (A 32 KB + B 32 KB).  Tiles that share their 256 tokens are adjacent in the walk, so the
// z tile is read from HBM once and from L2 by the other D/256 - 1 CTAs.
// (Loading the z tile with ordinary 16-byte loads into registers instead cost 37 L1 wavefronts per
// load instruction and left the kernel bound by the load/store unit at 1.23 ms for the d20 shape,
// against 0.66 ms with the TMA load.  Six stages of 32 columns with the 64-byte swizzle were no faster
// than three of 64 and doubled the L2 traffic; squaring one K step (16 columns) at a time, with a barrier
// per step so that its MMAs start early, was slower: 0.71 against 0.68 ms.  So was a ReLU^2 variant with
// the squared tile in tensor memory (128-token tiles, accumulator in 256 columns, A ring in the rest; no
// stores back to shared memory and no A reads from it): 0.72 ms, because a 128 x 256 tile needs 48 KB
// from L2 per 4.2 MFLOP against 64 KB per 8.4 MFLOP here, and both kernels take in about 90 GB/s per
// SM, which looks like the limit of the L2-to-SM path.)
#include <cuda.h>
#include <cudaTypedefs.h>

#include "skv_tc_common.cuh"

namespace skv {
namespace tc {

constexpr int32_t kStatusTimeoutReadout = 0x10;

namespace {

constexpr int kRoK = 64;                         // K columns per stage: 64 (128-byte swizzle) or 32 (64-byte swizzle)
constexpr int kRoStages = 192 / kRoK;            // 192 KB of stages
constexpr uint32_t kRoABytes = 256 * kRoK * 2;   // one A stage: 256 tokens x kRoK
constexpr uint32_t kRoBBytes = 256 * kRoK * 2;   // one B stage: 256 outputs x kRoK
constexpr int kRoThreads = 320;

struct RoParams {
  const uint8_t* wimg;           // [n_tiles][ks][kRoBBytes]
  __nv_bfloat16* y;
  int64_t ys;
  int64_t N;
  int h, r, D;
  int ks_z;                      // stages that read z: ceil(h / 32)
  int ks;                        // all stages: ks_z + ceil(r / 32)
  int n_tiles;                   // ceil(D / 256)
  int64_t tiles;                 // m_tiles * n_tiles
  int32_t* status;
  long long wait_cycles;
  int skip_copy;                 // test hook: the loader leaves out its first stage
};

// W[D][ws] (the layout of torch.nn.Linear.weight, columns [0,h) for act(z) and [h,h+r) for delta) ->
// per (output tile, stage) a 256 x kRoK K-major tile of 8 x 16-byte core matrices, [k core][n core][8 rows],
// zero where the tile reaches past D, h or r.
__global__ void tc_pack_w_kernel(const __nv_bfloat16* __restrict__ W, int64_t ws, int D, int h, int r, int ks_z, int ks,
                                 int64_t chunks, uint4* __restrict__ img) {
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < chunks; idx += (int64_t)gridDim.x * blockDim.x) {
    constexpr int kPer = (int)(kRoBBytes / 16);
    const int c = (int)(idx % kPer);
    const int64_t ts = idx / kPer;
    const int s = (int)(ts % ks);
    const int64_t nt = ts / ks;
    const int kc = c >> 8, nc = (c >> 3) & 31, row = c & 7;
    const int64_t n = nt * 256 + nc * 8 + row;
    bool ok = n < D;
    int64_t k;
    if (s < ks_z) {
      k = (int64_t)s * kRoK + kc * 8;
      ok = ok && k < h;
    } else {
      const int kd = (s - ks_z) * kRoK + kc * 8;
      ok = ok && kd < r;
      k = (int64_t)h + kd;
    }
    img[idx] = ok ? __ldg(reinterpret_cast<const uint4*>(W + n * ws + k)) : make_uint4(0, 0, 0, 0);
  }
}

__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Tiled TMA load, to this CTA alone, of one box of `map` at element coordinates (x, y) into this CTA's shared
// memory; x * 2 bytes is a multiple of 16 at every call site (x is a multiple of 64).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

template <bool RELU>
__global__ void __launch_bounds__(kRoThreads, 1)
    tc_readout_kernel(const RoParams P, const __grid_constant__ CUtensorMap map_z, const __grid_constant__ CUtensorMap map_d) {
  extern __shared__ uint8_t smem_raw[];
  // the swizzled A stages need 512-byte alignment (1024 keeps room for the 128-byte mode)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* a_base = smem;
  uint8_t* b_base = smem + kRoStages * kRoABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_base + kRoStages * kRoBBytes);
  uint64_t* full = bars;                         // [stages] TMA + bulk copy landed
  uint64_t* ready = full + kRoStages;            // [stages] activation applied (one arrival per warp); RELU only
  uint64_t* empty = ready + kRoStages;           // [stages] MMA -> loader
  uint64_t* acc_full = empty + kRoStages;        // [1] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 1;            // [1] epilogue -> MMA (one arrival per warp)
  uint64_t* done = acc_empty + 1;                // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutReadout, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < kRoStages; ++i) { mbar_init(full + i, 1); mbar_init(ready + i, 8); mbar_init(empty + i, 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 8) tmem_alloc(tmem_slot, 512);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int64_t step = gridDim.x;

  if (warp < 8) {
    // ------------------------------------------------------------------ activation in place, then epilogue
    uint32_t it = 0, ti = 0;
    bool drain = false;
    for (int64_t t = blockIdx.x; t < P.tiles && !drain; t += step, ++ti) {
      if (RELU) {
        for (int s = 0; s < P.ks && !drain; ++s, ++it) {
          const uint32_t st = it % kRoStages;
          if (mbar_wait(full + st, (it / kRoStages) & 1u, wc)) { drain = true; break; }
          if (s < P.ks_z) {
            // elementwise, so the swizzled layout does not matter: 16-byte chunk j * 256 + tid of the stage
            constexpr int kPerThread = (int)(kRoABytes / 4096);
            const uint32_t src = smem_u32(a_base + st * kRoABytes) + (uint32_t)tid * 16u;
            uint4 v[kPerThread];
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) v[j] = lds128(src + (uint32_t)j * 4096u);
#pragma unroll
            for (int j = 0; j < kPerThread; ++j) {
              v[j].x = relu_sq_bf2(v[j].x); v[j].y = relu_sq_bf2(v[j].y);
              v[j].z = relu_sq_bf2(v[j].z); v[j].w = relu_sq_bf2(v[j].w);
              sts128(src + (uint32_t)j * 4096u, v[j]);
            }
            fence_async_smem();
          }
          mbar_arrive_warp(ready + st);
        }
        if (drain) break;
      }
      // ---- epilogue of this tile: accumulator rows of this warp -> bf16 -> y
      if (mbar_wait(acc_full, ti & 1u, wc)) break;
      tc_fence_after();
      const int64_t n = (t / P.n_tiles) * 256 + warp * 32 + lane;
      const int n0 = (int)(t % P.n_tiles) * 256;
      const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(warp >> 2) * 256u;
      __nv_bfloat16* yrow = P.y + (n < P.N ? n : 0) * P.ys + n0;
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        float v[32];
        tmem_ld16(taddr + (uint32_t)(c * 32), v);
        tmem_ld16(taddr + (uint32_t)(c * 32 + 16), v + 16);
        if (n < P.N) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = c * 32 + q * 8;
            if (n0 + col < P.D)
              *reinterpret_cast<uint4*>(yrow + col) =
                  make_uint4(pack_bf2(v[q * 8], v[q * 8 + 1]), pack_bf2(v[q * 8 + 2], v[q * 8 + 3]),
                             pack_bf2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf2(v[q * 8 + 6], v[q * 8 + 7]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive_warp(acc_empty);
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      // A: K-major tile whose rows are one swizzle span (128 or 64 bytes) long, 8-row groups 8 rows apart;
      // a K step of 16 elements advances the start address by 32 bytes inside the swizzled row.
      constexpr uint32_t kRowBytes = kRoK * 2;
      const uint32_t a_hi = ((8u * kRowBytes) >> 4) | (1u << 14) | ((kRoK == 64 ? 2u : 4u) << 29);
      const uint32_t b_hi = desc_hi(128u);
      constexpr uint32_t idesc = instr_desc(1, 1, 0, 0, 128, 256);
      uint32_t it = 0, ti = 0;
      bool drain = false;
      for (int64_t t = blockIdx.x; t < P.tiles && !drain; t += step, ++ti) {
        if (ti >= 1) drain = mbar_wait(acc_empty, (ti - 1u) & 1u, wc);
        if (drain) break;
        tc_fence_after();
        for (int s = 0; s < P.ks; ++s, ++it) {
          const uint32_t st = it % kRoStages, ph = (it / kRoStages) & 1u;
          drain = mbar_wait((RELU ? ready : full) + st, ph, wc);
          if (drain) break;
          tc_fence_after();
          int nk = kRoK / 16;
          if (s >= P.ks_z) nk = min(kRoK / 16, (P.r - (s - P.ks_z) * kRoK + 15) / 16);
          uint32_t a_lo = ((smem_u32(a_base + st * kRoABytes) >> 4) & 0x3FFFu) | (1u << 16);
          uint32_t b_lo = desc_lo(smem_u32(b_base + st * kRoBBytes), 4096u);
          for (int k = 0; k < nk; ++k) {
            const uint32_t accf = (s | k) ? 1u : 0u;
            umma_f16_split(tmem_base, a_lo, a_hi, b_lo, b_hi, idesc, accf);                        // tokens 0-127
            umma_f16_split(tmem_base + 256u, a_lo + ((128u * kRowBytes) >> 4), a_hi, b_lo, b_hi, idesc, accf);  // tokens 128-255
            a_lo += 32u >> 4;
            b_lo += 8192u >> 4;
          }
          umma_commit(empty + st);
        }
        if (!drain) umma_commit(acc_full);
      }
      umma_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      uint32_t it = 0;
      bool stop = false;
      for (int64_t t = blockIdx.x; t < P.tiles && !stop; t += step) {
        const uint8_t* src = P.wimg + (size_t)(t % P.n_tiles) * P.ks * kRoBBytes;
        const int m0 = (int)((t / P.n_tiles) * 256);
        for (int s = 0; s < P.ks; ++s, ++it) {
          const uint32_t st = it % kRoStages;
          if (it == 0 && P.skip_copy) continue;      // test hook: nothing ever completes full[0]
          if (it >= kRoStages && mbar_wait(empty + st, ((it / kRoStages) - 1u) & 1u, wc)) { stop = true; break; }
          mbar_arrive_expect_tx(full + st, kRoABytes + kRoBBytes);
          if (s < P.ks_z) tma_load_2d(a_base + st * kRoABytes, &map_z, s * kRoK, m0, full + st);
          else tma_load_2d(a_base + st * kRoABytes, &map_d, (s - P.ks_z) * kRoK, m0, full + st);
          bulk_g2s(b_base + st * kRoBBytes, src + (size_t)s * kRoBBytes, kRoBBytes, full + st);
        }
      }
      if (*abort_flag) {              // let copies in flight land before the CTA's shared memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    mbar_wait_drain(done, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, 512);
  }
}

PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Map of a [rows][cols] bf16 matrix with row pitch `pitch` elements; boxes of 256 rows x kRoK columns,
// the swizzle span of one row, zeros outside the matrix.
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch) {
  PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
  if (!enc) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch * 2};
  const cuuint32_t box[2] = {kRoK, 256};
  const cuuint32_t es[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, kRoK == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool readout_eligible(const skv_problem& p, int64_t D) {
  return p.N < ((int64_t)1 << 31) - 256 && p.dtype == SKV_BF16 && (p.activation == SKV_ACT_RELU_SQ || p.activation == SKV_ACT_IDENTITY) && p.h % 8 == 0 &&
         p.r % 8 == 0 && D >= 8 && D % 8 == 0 && D <= (1 << 24);
}

size_t readout_image_bytes(const skv_problem& p, int64_t D) {
  const size_t ks = (size_t)(p.h + kRoK - 1) / kRoK + (size_t)(p.r + kRoK - 1) / kRoK;
  return (size_t)((D + 255) / 256) * ks * kRoBBytes;
}

// Row pitch (elements) of the delta buffer the GEMM reads: whole stages of kRoK columns, pad columns zero.
int64_t readout_delta_pitch(const skv_problem& p) { return (int64_t)((p.r + kRoK - 1) / kRoK) * kRoK; }

// y = [act(z) | delta] * W^T; `delta` is [N][readout_delta_pitch()] bf16 with zero pad columns, `wimg`
// has readout_image_bytes().
int readout(const LaunchCtx& c, const void* z, int64_t zs, const void* delta, const void* W, int64_t ws, int64_t D,
            void* y, int64_t ys, void* wimg) {
  const skv_problem& p = c.p;
  RoParams P;
  P.wimg = static_cast<const uint8_t*>(wimg);
  P.y = static_cast<__nv_bfloat16*>(y);
  P.ys = ys;
  P.N = p.N;
  P.h = (int)p.h;
  P.r = (int)p.r;
  P.D = (int)D;
  P.ks_z = (int)((p.h + kRoK - 1) / kRoK);
  P.ks = P.ks_z + (int)((p.r + kRoK - 1) / kRoK);
  P.n_tiles = (int)((D + 255) / 256);
  P.tiles = ((p.N + 255) / 256) * P.n_tiles;
  P.status = c.status;
  P.wait_cycles = wait_cycle_limit();
  P.skip_copy = debug_skip_copy() == 2;
  CUtensorMap map_z, map_d;
  if (!make_map(&map_z, z, (uint64_t)p.N, (uint64_t)p.h, (uint64_t)zs) ||
      !make_map(&map_d, delta, (uint64_t)p.N, (uint64_t)readout_delta_pitch(p), (uint64_t)readout_delta_pitch(p)))
    return SKV_ERR_LAUNCH;

  const int64_t chunks = (int64_t)P.n_tiles * P.ks * (kRoBBytes / 16);
  const int pgrid = (int)((chunks + 255) / 256 < 4096 ? (chunks + 255) / 256 : 4096);
  tc_pack_w_kernel<<<pgrid, 256, 0, c.stream>>>(static_cast<const __nv_bfloat16*>(W), ws, P.D, P.h, P.r, P.ks_z, P.ks,
                                                 chunks, static_cast<uint4*>(wimg));
  if (cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;

  const size_t smem = (size_t)kRoStages * (kRoABytes + kRoBBytes) + 1024 + 256;
  const int grid = (int)(P.tiles < c.num_sms ? P.tiles : c.num_sms);
  cudaError_t err;
  if (p.activation == SKV_ACT_RELU_SQ) {
    err = cudaFuncSetAttribute(tc_readout_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err == cudaSuccess) tc_readout_kernel<true><<<grid, kRoThreads, smem, c.stream>>>(P, map_z, map_d);
  } else {
    err = cudaFuncSetAttribute(tc_readout_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err == cudaSuccess) tc_readout_kernel<false><<<grid, kRoThreads, smem, c.stream>>>(P, map_z, map_d);
  }
  if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) return SKV_ERR_LAUNCH;
  note_launches(2);
  return SKV_OK;
}

}  // namespace tc
}  // namespace skv
