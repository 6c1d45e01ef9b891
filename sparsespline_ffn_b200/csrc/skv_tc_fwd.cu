// tcgen05 forward of the spline-KV feature operator (bf16 I/O, r a multiple of 16 up to 128,
// h a multiple of 8).
//
//   delta[n, c] = sum_j sum_b Phi[n, (j,b)] * C[j, b, c]
//
// is computed as a dense GEMM on the 5th-generation tensor cores: the expanded basis Phi (three
// non-zero weights per key, at knot rows bin..bin+2) is built per token as f16, the code table is
// staged by TMA bulk copies from a range-scaled f16 image in the canonical operand layout, and
// tcgen05.mma accumulates 128-token x r tiles in tensor memory in float32.  A small second kernel
// sums the key splits, applies lambda and casts.
//
// Two kernels.  tc_forward_ta_kernel (the one used for the knot counts in common use) keeps Phi
// in tensor memory: every producer thread builds the complete row segment of a key in registers
// and writes it into its own tensor-memory lane, and the MMA takes its A operand from there.
// tc_forward_kernel keeps Phi in shared memory (scattered 32-bit stores, bound by shared-memory
// bandwidth) and serves the remaining knot counts.  Their launch shapes and warp roles are
// described at each kernel.
//
// A key with an odd number of knot rows is padded by one zero row in the operand images.
// Every mbarrier wait is bounded (skv_tc_common.cuh); a timed-out wait sets the status word and
// lets the CTA drain.
#include "skv_tc_common.cuh"

namespace skv {
namespace tc {
namespace {

constexpr int kStages = 2;
constexpr int kMaxCStages = 4;
constexpr int kMaxTaCStages = 8;
constexpr int kChunkKeys = 8;
constexpr int kPlanSMs = 148;                 // B200; only used to balance the launch shape
constexpr size_t kSmemLimit = 227 * 1024;

struct FwdParams {
  const __nv_bfloat16* z;
  int64_t zs;
  __nv_bfloat16* act_out;
  int64_t as;
  const __half* cimg;       // [h/8][8L/8][r/8][8][8] f16 image of C
  float* partial;           // [splits][N][r]
  int64_t N;
  int h, L, r;
  int LR;                   // knot rows per key in the shared-memory Phi tile: L rounded up to even
  GridParams g;
  int act;
  int chunks_total, chunks_per_split;
  int32_t* status;
  uint32_t a_lbo, a_sbo, b_lbo, b_sbo;
  int cstages;              // depth of the code-table ring (2..4)
  long long wait_cycles;     // limit of every bounded wait, in clock cycles
  int skip_copy;             // test hook: the loader leaves out the copy of its first chunk
};

// Phi in shared memory.  Launch shape: grid = (token tiles of 128*GROUPS tokens, key splits).  A CTA
// walks its keys in chunks of 8 (K extent 8*LR per chunk) through a two-stage ring:
//   warps 0..4*GROUPS-1  producers, one thread per token: read 8 pre-activations, write the
//                        phi(z) half of the output, compute knot interval and weights in
//                        registers, store the two non-zero 32-bit words of the Phi row segment;
//                        after the last chunk they read the accumulator from tensor memory and
//                        store the float32 partial residual of this key split
//   warp 4*GROUPS        lane 0 issues the MMAs of each chunk and commits to the ring barriers
//   warp 4*GROUPS+1      lane 0 issues the bulk copies of the code-table image
template <int GROUPS>
__global__ void __launch_bounds__(128 * GROUPS + 64, 1) tc_forward_kernel(const FwdParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int L = P.LR, r = P.r;                                    // padded rows: the pad row stays zero
  const uint32_t phi_bytes = (uint32_t)L * 2048u;                 // 128 tokens x 8L f16
  const uint32_t c_bytes = (uint32_t)(kChunkKeys * L * r * 2);
  uint8_t* phi_base = smem;                                        // [stage][group][phi_bytes]
  const int CS = P.cstages;
  uint8_t* c_base = smem + (size_t)kStages * GROUPS * phi_bytes;   // [cstage][c_bytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(c_base + (size_t)CS * c_bytes);
  uint64_t* full = bars;                          // [stage][group]   producers -> MMA
  uint64_t* empty = full + kStages * GROUPS;      // [stage][group]   MMA -> producers
  uint64_t* cfull = empty + kStages * GROUPS;     // [cstage]         TMA -> MMA
  uint64_t* cempty = cfull + kMaxCStages;         // [cstage]         MMA -> TMA
  uint64_t* done = cempty + kMaxCStages;          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutFwd, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk_begin = blockIdx.y * P.chunks_per_split;
  const int nch = min(P.chunks_per_split, P.chunks_total - chunk_begin);
  const int64_t tile_base = (int64_t)blockIdx.x * (128 * GROUPS);
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)(GROUPS * r)) tmem_cols <<= 1;

  if (tid == 0) {
    for (int i = 0; i < kStages * GROUPS; ++i) { mbar_init(full + i, 4); mbar_init(empty + i, 1); }
    for (int i = 0; i < kMaxCStages; ++i) { mbar_init(cfull + i, 1); mbar_init(cempty + i, 1); }
    mbar_init(done, 1);
    *abort_flag = 0;
    mbar_init_fence();
  }
  // zero both Phi stages once; afterwards producers clear exactly the words they wrote
  {
    uint4* p = reinterpret_cast<uint4*>(phi_base);
    const uint32_t n16 = kStages * GROUPS * phi_bytes / 16;
    for (uint32_t i = tid; i < n16; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
  }
  if (warp == 4 * GROUPS) tmem_alloc(tmem_slot, tmem_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4 * GROUPS) {
    // ------------------------------------------------------------------ producers / epilogue
    const int grp = warp >> 2;
    const int t = tid & 127;
    const int64_t n = tile_base + grp * 128 + t;
    const bool valid = n < P.N;
    const uint32_t t_off = (uint32_t)(t & 7) * 16u + (uint32_t)(t >> 3) * 128u;
    const __nv_bfloat16* zrow = P.z + (valid ? n : 0) * P.zs + (int64_t)chunk_begin * kChunkKeys;
    __nv_bfloat16* arow = P.act_out ? P.act_out + (valid ? n : 0) * P.as + (int64_t)chunk_begin * kChunkKeys : nullptr;
    const uint32_t halfL = (uint32_t)L >> 1;
    uint32_t saved[kStages][kChunkKeys];
#pragma unroll
    for (int i = 0; i < kStages; ++i)
#pragma unroll
      for (int q = 0; q < kChunkKeys; ++q) saved[i][q] = 0;
    uint4 znext = valid && nch > 0 ? __ldg(reinterpret_cast<const uint4*>(zrow)) : make_uint4(0, 0, 0, 0);
    const int act = P.act;

    auto chunk_body = [&](int ci, int s, uint32_t(&sv)[kChunkKeys]) {
      const uint4 zc = znext;
      if (ci + 1 < nch && valid) znext = __ldg(reinterpret_cast<const uint4*>(zrow + (ci + 1) * kChunkKeys));
      const uint32_t row = smem_u32(phi_base + (size_t)(s * GROUPS + grp) * phi_bytes) + t_off;
      if (ci >= kStages) {
        mbar_wait(empty + s * GROUPS + grp, (uint32_t)((ci / kStages) - 1) & 1u, wc);
        if (valid) {
#pragma unroll
          for (int q = 0; q < kChunkKeys; ++q) {
            sts32(row + (sv[q] & 0xffffu) * 4u, 0u);
            sts32(row + (sv[q] >> 16) * 4u, 0u);
          }
        }
      }
      if (valid) {
        const uint32_t zw[4] = {zc.x, zc.y, zc.z, zc.w};
        uint32_t aw[4];
#pragma unroll
        for (int q = 0; q < kChunkKeys; ++q) {
          const float zz = (q & 1) ? bf_hi(zw[q >> 1]) : bf_lo(zw[q >> 1]);
          uint32_t x0, x1, wo0, wo1;
          phi_pair(zz, P.g, (uint32_t)q * halfL, x0, x1, wo0, wo1);
          sts32(row + wo0 * 4u, x0);
          sts32(row + wo1 * 4u, x1);
          sv[q] = wo0 | (wo1 << 16);
          const float a = act_fwd(zz, act);
          if (q & 1) aw[q >> 1] = pack_bf2(__uint_as_float(aw[q >> 1]), a);
          else aw[q >> 1] = __float_as_uint(a);
        }
        if (arow) *reinterpret_cast<uint4*>(arow + ci * kChunkKeys) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
      }
      fence_async_smem();
      mbar_arrive_warp(full + s * GROUPS + grp);
    };

    for (int ci = 0; ci < nch; ci += kStages) {
      chunk_body(ci, 0, saved[0]);
      if (ci + 1 < nch) chunk_body(ci + 1, 1, saved[1]);
    }

    // epilogue: accumulator -> float32 partial of this key split
    mbar_wait(done, 0, wc);
    tc_fence_after();
    float* prow = P.partial + ((size_t)blockIdx.y * P.N + (valid ? n : 0)) * r;
    const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(grp * r);
    for (int c0 = 0; c0 < r; c0 += 16) {
      float v[16];
      tmem_ld16(taddr + c0, v);
      if (valid) {
#pragma unroll
        for (int i = 0; i < 16; i += 4)
          *reinterpret_cast<float4*>(prow + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      }
    }
    tc_fence_before();
  } else if (warp == 4 * GROUPS) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t idesc = instr_desc(0, 0, 0, 1, 128, r);
      const int ksteps = kChunkKeys * L / 16;
      const uint32_t a_hi = desc_hi(P.a_sbo), b_hi = desc_hi(P.b_sbo);
      const uint32_t a_step = (2u * 2048u) >> 4, b_step = (2u * (uint32_t)(r / 8) * 128u) >> 4;   // per K=16 step
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % kStages;
        const uint32_t par = (uint32_t)(ci / kStages) & 1u;
        const int cs = ci % CS;
        bool drain = mbar_wait(cfull + cs, (uint32_t)(ci / CS) & 1u, wc);
        const uint32_t b_lo0 = desc_lo(smem_u32(c_base + (size_t)cs * c_bytes), P.b_lbo);
        for (int grp = 0; grp < GROUPS && !drain; ++grp) {
          drain = mbar_wait(full + s * GROUPS + grp, par, wc);
          if (drain) break;                          // draining: issue nothing more
          tc_fence_after();
          uint32_t a_lo = desc_lo(smem_u32(phi_base + (size_t)(s * GROUPS + grp) * phi_bytes), P.a_lbo);
          uint32_t b_lo = b_lo0;
          const uint32_t d_addr = tmem_base + (uint32_t)(grp * r);
          umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, ci > 0 ? 1u : 0u);
          for (int ks = 1; ks < ksteps; ++ks) {
            a_lo += a_step;
            b_lo += b_step;
            umma_f16_split(d_addr, a_lo, a_hi, b_lo, b_hi, idesc, 1u);
          }
          umma_commit(empty + s * GROUPS + grp);
        }
        if (drain) break;
        umma_commit(cempty + cs);
      }
      umma_commit(done);
    }
  } else {
    // ------------------------------------------------------------------ code-table loader
    if (lane == 0) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(P.cimg) + (size_t)chunk_begin * c_bytes;
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % CS;
        if (ci >= CS)
          mbar_wait(cempty + s, (uint32_t)((ci / CS) - 1) & 1u, wc);
        if (*abort_flag) break;
        if (ci == 0 && P.skip_copy) continue;      // test hook: nothing ever completes cfull[0]
        mbar_arrive_expect_tx(cfull + s, c_bytes);
        bulk_g2s(c_base + (size_t)s * c_bytes, src + (size_t)ci * c_bytes, c_bytes, cfull + s);
      }
      // all copies issued have been consumed by the MMA warp unless the CTA is draining after a
      // timeout; in that case give copies still in flight time to land before the CTA exits
      if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
  }
  __syncthreads();
  if (warp == 4 * GROUPS) {
    // the accumulator has been read (or the CTA is draining): make sure no MMA is still running
    mbar_wait_drain(done, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------------------------
// Forward with the expanded basis held in tensor memory instead of shared memory.
//
// The shared-memory variant above is bound by shared-memory bandwidth: every MMA re-reads its
// 4 KB A tile while the producers scatter words into the same banks.  Here each producer thread
// builds the complete Phi row segment of a key (HL = L/2 f16x2 words, two of them non-zero) in
// registers and writes it with tcgen05.st into its own tensor-memory lane; the MMA takes A from
// tensor memory and only the code-table chunk (B) from shared memory.  Nothing has to be
// cleared: a row segment is overwritten completely every chunk.
//
// Tensor-memory columns per token group: 8*HL for A (single-buffered) followed by r for the
// accumulator; with four groups (512 tokens per CTA, 16 producer warps) the other groups keep the
// SM busy while one group waits for its MMAs.
// ---------------------------------------------------------------------------------------------
// Keys of each half chunk (of four) that are placed through the staging row (load/store pipe); the
// others are placed by multiplying with 0/1 masks in packed f16 arithmetic (FMA pipe).  When the
// others used compare/select chains (ALU pipe, which issues at half rate and was 66 % busy) two of
// four was the balance: 1 -> 1.07 ms, 2 -> 0.95 ms, 3 -> 0.99 ms, 4 -> 1.11 ms at the d20 shape.  With
// the mask arithmetic: 0 -> 0.955 ms, 1 -> 0.900 ms, 2 -> 0.908 ms, 3 -> 0.984 ms (0.917 / 0.890 / 0.903
// for 0 / 1 / 2 once two keys share their tensor-memory stores).
#ifndef SKV_NSTH
#define SKV_NSTH 1
#endif
constexpr int kStagedPerHalf = SKV_NSTH;

template <int GROUPS, int HL, int ACT, int NSTH>
__global__ void __launch_bounds__(160 * GROUPS + 32, 1) tc_forward_ta_kernel(const FwdParams P) {
  extern __shared__ __align__(128) uint8_t smem[];
  // Keys are padded to HLP words (an even count), so that half a chunk (4 keys) is a whole number
  // of K = 16 steps; the code-table image has 2*HLP rows per key, the padding rows are zero.
  constexpr int HLP = (HL + 1) & ~1;
  constexpr int kHalfKeys = kChunkKeys / 2;
  constexpr int kHalfSteps = kHalfKeys * HLP / 8;                  // K = 16 steps per half chunk
  const int r = P.r;
  const uint32_t c_bytes = (uint32_t)(kChunkKeys * 2 * HLP * r * 2);
  const int CS = P.cstages;
  uint8_t* c_base = smem;                                          // [cstage][c_bytes]
  // One private staging row of HLP words per producer thread.  Placing the two non-zero words of
  // a row segment costs about thirty compare/select instructions on the half-rate ALU pipe; for
  // NSTH of the four keys of every half chunk the thread instead stores the two words into its
  // (zeroed) staging row at the dynamic position, reads the row back and zeroes the two words
  // again, which moves that work to the load/store pipe.  The rows of a warp are interleaved by
  // lane (word w of lane l at (w * 32 + l) * 4 bytes of the warp's region), so the bank of every
  // access is the lane and neither the scattered stores nor the loads conflict, whatever the knot
  // intervals of the 32 tokens are.
  constexpr int SW = HLP;
  uint8_t* stage_base = c_base + (size_t)CS * c_bytes;             // [128*GROUPS][SW words]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_base + (size_t)128 * GROUPS * SW * 4);
  uint64_t* full = bars;                          // [group][half]  producers -> MMA
  uint64_t* empty = full + 2 * GROUPS;            // [group][half]  MMA -> producers
  uint64_t* cfull = empty + 2 * GROUPS;           // [cstage]       TMA -> MMA
  uint64_t* cempty = cfull + kMaxTaCStages;       // [cstage]       MMA -> TMA
  uint64_t* done = cempty + kMaxTaCStages;        // [group]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + GROUPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wc{abort_flag, P.status, kStatusTimeoutFwd, P.wait_cycles};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk_begin = blockIdx.y * P.chunks_per_split;
  const int nch = min(P.chunks_per_split, P.chunks_total - chunk_begin);
  const int64_t tile_base = (int64_t)blockIdx.x * (128 * GROUPS);
  const uint32_t grp_cols = (uint32_t)(kChunkKeys * HLP + r);
  uint32_t tmem_cols = 32;
  while (tmem_cols < GROUPS * grp_cols) tmem_cols <<= 1;

  if (tid == 0) {
    for (int i = 0; i < 2 * GROUPS; ++i) { mbar_init(full + i, 4); mbar_init(empty + i, 1); }
    for (int i = 0; i < GROUPS; ++i) mbar_init(done + i, 1);
    for (int i = 0; i < kMaxTaCStages; ++i) { mbar_init(cfull + i, 1); mbar_init(cempty + i, GROUPS); }
    *abort_flag = 0;
    mbar_init_fence();
  }
  for (uint32_t i = tid; i < (uint32_t)(128 * GROUPS * SW / 4); i += blockDim.x)
    reinterpret_cast<uint4*>(stage_base)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 5 * GROUPS) tmem_alloc(tmem_slot, tmem_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4 * GROUPS) {
    // ------------------------------------------------------------------ producers / epilogue
    const int grp = warp >> 2;
    const int t = tid & 127;
    const int64_t n = tile_base + grp * 128 + t;
    const bool valid = n < P.N;
    const __nv_bfloat16* zrow = P.z + (valid ? n : 0) * P.zs + (int64_t)chunk_begin * kChunkKeys;
    __nv_bfloat16* arow = P.act_out ? P.act_out + (valid ? n : 0) * P.as + (int64_t)chunk_begin * kChunkKeys : nullptr;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)grp * grp_cols;
    uint4 znext = valid && nch > 0 ? __ldg(reinterpret_cast<const uint4*>(zrow)) : make_uint4(0, 0, 0, 0);
    // word w of this thread's staging row lives at (warp * HLP + w) * 128 + lane * 4: its bank is the
    // lane, whatever w is, so neither the scattered stores nor the loads conflict
    const uint32_t srow = smem_u32(stage_base) + (uint32_t)(warp * HLP * 128 + lane * 4);
    const uint32_t srow_biased = srow - (kWordBias << 7);          // wp carries the bias kWordBias
    for (int ci = 0; ci < nch; ++ci) {
      const uint4 zc = znext;
      if (ci + 1 < nch && valid) znext = __ldg(reinterpret_cast<const uint4*>(zrow + (ci + 1) * kChunkKeys));
      const uint32_t zw[4] = {zc.x, zc.y, zc.z, zc.w};
      // phi(z) of the chunk's eight keys in packed bf16 arithmetic: the product of two bf16 values is
      // exact in float32, so one rounding to bf16 gives the same result as float32 arithmetic and a cast
      uint32_t aw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (ACT == SKV_ACT_RELU_SQ) aw[i] = relu_sq_bf2(zw[i]);
        else if constexpr (ACT == SKV_ACT_GELU) aw[i] = pack_bf2(gelu_fwd(bf_lo(zw[i])), gelu_fwd(bf_hi(zw[i])));
        else aw[i] = zw[i];
      }
      // The group's A columns are written and consumed in two halves of 4 keys: the MMAs of one
      // half run while the other half is being built, so the producers do not wait for them.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (ci > 0) {
          mbar_wait(empty + grp * 2 + half, (uint32_t)(ci - 1) & 1u, wc);
          tc_fence_after();
        }
        // The first NSTH keys of the half go through the staging row: their stores and loads are
        // issued first, the select chains of the other keys run while those loads are in flight,
        // and the staged rows are written to tensor memory last.
        // The words of two neighbouring keys are stored to tensor memory together (2 * HLP columns:
        // one 16- and one 8-column store at HLP = 12 instead of two of each).
        uint32_t WP[kHalfKeys / 2][2 * HLP];
        // knot interval and weights of the half's four keys, two keys (one packed z word) at a time
        uint32_t kx0[kHalfKeys], kx1[kHalfKeys], kwp[kHalfKeys];
#pragma unroll
        for (int pq = 0; pq < kHalfKeys / 2; ++pq) {
          uint32_t a0[2], a1[2], aw2[2];
          phi_pair_words2(zw[half * (kHalfKeys / 2) + pq], P.g, a0, a1, aw2);   // rows past N read z = 0; their accumulator rows are never stored
          kx0[2 * pq] = a0[0]; kx1[2 * pq] = a1[0]; kwp[2 * pq] = aw2[0];
          kx0[2 * pq + 1] = a0[1]; kx1[2 * pq + 1] = a1[1]; kwp[2 * pq + 1] = aw2[1];
        }
#pragma unroll
        for (int qq = 0; qq < NSTH; ++qq) {
          const uint32_t x0 = kx0[qq], x1 = kx1[qq], wp = kwp[qq];
          const uint32_t pos = srow_biased + (wp << 7);
          sts32(pos, x0);
          sts32(pos + 128u, x1);
#pragma unroll
          for (int i = 0; i < HLP; ++i)
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(WP[qq >> 1][(qq & 1) * HLP + i]) : "r"(srow + (uint32_t)i * 128u) : "memory");
          sts32(pos, 0u);
          sts32(pos + 128u, 0u);
        }
#pragma unroll
        for (int qq = NSTH; qq < kHalfKeys; ++qq) {
          const uint32_t x0 = kx0[qq], x1 = kx1[qq], wp = kwp[qq];
          // Placement at word-pair granularity: wp = 2 * qd + s.  The two words land in pair qd as
          // (x0, x1) when s = 0, or as (0, x0) there and (x1, 0) in pair qd + 1 when s = 1.
          uint32_t* W = &WP[qq >> 1][(qq & 1) * HLP];
          const bool odd = (wp & 1u) != 0u;
          const uint32_t y0 = odd ? 0u : x0, y1 = odd ? x0 : x1, y2 = odd ? x1 : 0u;
          constexpr int kLastPair = (HL - 2) >> 1;               // largest qd: bin <= L - 3
          // Each word is its value times a 0/1 mask in packed f16 arithmetic (x * 1 and x * 0 are exact
          // for the non-negative finite weights, and at most one term of a sum is non-zero), so the
          // placement runs on the FMA pipe instead of compare/select chains on the busier ALU pipe.
          // wp >> 1 is (kKnotBias >> 2) + qd with qd < 64; times 0x10001 that is the f16 pair with bit
          // patterns qd (low: a subnormal, or zero) and (kKnotBias >> 18) + qd (high): distinct per qd.
          // f16 comparisons do not flush subnormals (this file is not built with a flush-to-zero flag).
          const uint32_t q2 = (wp >> 1) * 0x00010001u;
          const __half2 qh = *reinterpret_cast<const __half2*>(&q2);
          const __half2 h0 = *reinterpret_cast<const __half2*>(&y0), h1 = *reinterpret_cast<const __half2*>(&y1),
                        h2 = *reinterpret_cast<const __half2*>(&y2);
          __half2 m[HLP / 2];
#pragma unroll
          for (int i = 0; i < HLP / 2; ++i) {
            const uint32_t ci2 = (((kKnotBias >> 18) + (uint32_t)i) << 16) | (uint32_t)i;
            m[i] = i <= kLastPair ? __heq2(qh, *reinterpret_cast<const __half2*>(&ci2)) : __float2half2_rn(0.0f);
          }
#pragma unroll
          for (int i = 0; i < HLP / 2; ++i) {
            __half2 e = __hmul2(m[i], h0);
            if (i > 0) e = __hfma2(m[i - 1], h2, e);
            const __half2 o = __hmul2(m[i], h1);
            W[2 * i] = *reinterpret_cast<const uint32_t*>(&e);
            W[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&o);
          }
          if ((qq & 1) && (qq & ~1) >= NSTH)            // a pair of mask-placed keys is complete
            tmem_st_words<2 * HLP>(lane_addr + (uint32_t)((half * kHalfKeys + (qq & ~1)) * HLP), WP[qq >> 1]);
        }
        // (All four keys in one 32- and one 16-column store was slower: 0.909 against 0.890 ms.)
#pragma unroll
        for (int pp = 0; 2 * pp < NSTH; ++pp)            // pairs with a staged key: their loads have landed by now
          tmem_st_words<2 * HLP>(lane_addr + (uint32_t)((half * kHalfKeys + 2 * pp) * HLP), WP[pp]);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive_warp(full + grp * 2 + half);
      }
      if (arow && valid) *reinterpret_cast<uint4*>(arow + ci * kChunkKeys) = make_uint4(aw[0], aw[1], aw[2], aw[3]);
    }
    // epilogue: accumulator -> float32 partial of this key split
    mbar_wait(done + grp, 0, wc);
    tc_fence_after();
    float* prow = P.partial + ((size_t)blockIdx.y * P.N + (valid ? n : 0)) * r;
    const uint32_t daddr = lane_addr + (uint32_t)(kChunkKeys * HLP);
    for (int c0 = 0; c0 < r; c0 += 16) {
      float v[16];
      tmem_ld16(daddr + c0, v);
      if (valid) {
#pragma unroll
        for (int i = 0; i < 16; i += 4)
          *reinterpret_cast<float4*>(prow + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      }
    }
    tc_fence_before();
  } else if (warp < 5 * GROUPS) {
    // ------------------------------------------------------------------ MMA issue, one warp per token group
    // (one thread cannot issue N = r MMAs faster than about one per 45 cycles)
    if (lane == 0) {
      const int grp = warp - 4 * GROUPS;
      const uint32_t idesc = instr_desc(0, 0, 0, 1, 128, r);
      const uint32_t b_hi = desc_hi(P.b_sbo);
      const uint32_t b_step = (2u * (uint32_t)(r / 8) * 128u) >> 4;          // per K=16 step
      const uint32_t a_addr0 = tmem_base + (uint32_t)grp * grp_cols;
      const uint32_t d_addr = a_addr0 + (uint32_t)(kChunkKeys * HLP);
      for (int ci = 0; ci < nch; ++ci) {
        const int cs = ci % CS;
        bool drain = mbar_wait(cfull + cs, (uint32_t)(ci / CS) & 1u, wc);
        uint32_t b_lo = desc_lo(smem_u32(c_base + (size_t)cs * c_bytes), P.b_lbo);
        uint32_t a_addr = a_addr0;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          drain = drain || mbar_wait(full + grp * 2 + half, (uint32_t)ci & 1u, wc);
          if (drain) break;                          // draining: issue nothing more
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kHalfSteps; ++ks) {     // 8 columns of A (16 K elements) per step
            umma_f16_ta(d_addr, a_addr, b_lo, b_hi, idesc, (ci > 0 || half > 0 || ks > 0) ? 1u : 0u);
            a_addr += 8u;
            b_lo += b_step;
          }
          umma_commit(empty + grp * 2 + half);
        }
        if (drain) break;
        umma_commit(cempty + cs);
      }
      umma_commit(done + grp);
    }
  } else {
    // ------------------------------------------------------------------ code-table loader
    if (lane == 0) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(P.cimg) + (size_t)chunk_begin * c_bytes;
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % CS;
        if (ci >= CS)
          mbar_wait(cempty + s, (uint32_t)((ci / CS) - 1) & 1u, wc);
        if (*abort_flag) break;
        if (ci == 0 && P.skip_copy) continue;      // test hook: nothing ever completes cfull[0]
        mbar_arrive_expect_tx(cfull + s, c_bytes);
        bulk_g2s(c_base + (size_t)s * c_bytes, src + (size_t)ci * c_bytes, c_bytes, cfull + s);
      }
      if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
  }
  __syncthreads();
  if (warp == 5 * GROUPS) {
    for (int i = 0; i < GROUPS; ++i) mbar_wait_drain(done + i, 0, P.wait_cycles);
    tc_fence_after();
    tmem_free(tmem_base, tmem_cols);
  }
}

// C [h][L][r] bf16 -> f16 image: per 8-key chunk the [8L x r] tile as 8x8 core matrices,
// core (kg, cg) at ((kg * r/8 + cg) * 128) bytes, row k%8 at 16 bytes, channel c%8 at 2 bytes.
__global__ void tc_pack_c_kernel(const __nv_bfloat16* __restrict__ C, __half* __restrict__ img, int h, int L, int LP,
                                 int r, const uint32_t* __restrict__ amax_bits) {
  float cscale, cinv;
  pow2_scales(amax_bits[kAmaxC], cscale, cinv);
  const int rows_per_chunk = kChunkKeys * LP;          // LP >= L rows per key in the image, rows L.. are zero
  const int cgs = r / 8;
  const size_t pieces = (size_t)h * LP * cgs;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (size_t)gridDim.x * blockDim.x) {
    const int cg = (int)(i % cgs);
    const size_t rowg = i / cgs;                       // (j, b) row of the padded image
    const int chunk = (int)(rowg / rows_per_chunk);
    const int k = (int)(rowg % rows_per_chunk);
    const int j = (int)(rowg / LP), bb = (int)(rowg % LP);
    const uint4 v = bb < L ? __ldg(reinterpret_cast<const uint4*>(C + ((size_t)j * L + bb) * r + cg * 8))
                           : make_uint4(0, 0, 0, 0);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) o[q] = pack_h2(bf_lo(w[q]) * cscale, bf_hi(w[q]) * cscale);
    __half* dst = img + (size_t)chunk * rows_per_chunk * r + ((size_t)(k >> 3) * cgs + cg) * 64 + (k & 7) * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <typename TD>
__global__ void tc_finalize_kernel(const float* __restrict__ partial, int splits, int64_t N, int r, float lambda,
                                   const uint32_t* __restrict__ amax_bits, TD* __restrict__ out, int64_t ds) {
  float cscale, cinv;
  pow2_scales(amax_bits[kAmaxC], cscale, cinv);
  lambda *= cinv;                                       // undo the code-table image's range scaling
  const int64_t total = N * r;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += partial[(size_t)k * total + i];
    st_f32<TD>(out + (i / r) * ds + (i % r), lambda * s);
  }
}


struct FwdPlan {
  int groups, splits, chunks_per_split, cstages;
  size_t smem;
  bool ta;                  // expanded basis in tensor memory (tc_forward_ta_kernel) instead of shared memory
};

// Half knot-row counts (L/2) the tensor-memory variant is instantiated for.
bool ta_supported_hl(int hl) { return hl == 8 || hl == 11 || hl == 12 || hl == 16 || hl == 21; }

size_t fwd_smem(int groups, int cstages, int L, int r) {
  return (size_t)kStages * groups * L * 2048 + (size_t)cstages * kChunkKeys * L * r * 2 + 256;
}

bool plan_forward(const skv_problem& p, FwdPlan* out) {
  out->ta = false;
  const int hl = (p.L + 1) / 2;                       // f16x2 words per key (an odd L leaves one half empty)
  const int hlp = (hl + 1) & ~1;                      // words per key in tensor memory (padded to even)
  if (ta_supported_hl(hl) && kChunkKeys * hlp + p.r <= 512) {
    int groups = 512 / (kChunkKeys * hlp + p.r);
    if (groups > 4) groups = 4;
    const size_t c_bytes = (size_t)kChunkKeys * 2 * hlp * p.r * 2;
    const int sw = hlp;                                            // staging-row words per producer thread
    const size_t stage_bytes = (size_t)128 * groups * sw * 4;
    int cstages = (int)((kSmemLimit - 512 - stage_bytes) / c_bytes);
    if (cstages > kMaxTaCStages) cstages = kMaxTaCStages;
    if (cstages >= 2) {
      out->ta = true;
      out->groups = groups;
      out->cstages = cstages;
      out->smem = (size_t)cstages * c_bytes + stage_bytes + 512;       // ring + staging rows + barriers
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
      out->chunks_per_split = (chunks + best - 1) / best;
      out->splits = (chunks + out->chunks_per_split - 1) / out->chunks_per_split;
      return true;
    }
  }
  const int LR = (p.L + 1) & ~1;
  int groups = 0;
  if (fwd_smem(2, 2, LR, p.r) <= kSmemLimit) groups = 2;
  else if (fwd_smem(1, 2, LR, p.r) <= kSmemLimit) groups = 1;
  if (!groups) return false;
  int cstages = 2;
  while (cstages < kMaxCStages && fwd_smem(groups, cstages + 1, LR, p.r) <= kSmemLimit) ++cstages;
  out->cstages = cstages;
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
  out->groups = groups;
  out->splits = best;
  out->chunks_per_split = (chunks + best - 1) / best;
  out->splits = (chunks + out->chunks_per_split - 1) / out->chunks_per_split;
  out->smem = fwd_smem(groups, cstages, LR, p.r);
  return true;
}

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace

bool fwd_eligible(const skv_problem& p) {
  if (p.dtype != SKV_BF16) return false;
  if (p.r % 16 || p.r < 16 || p.r > 128) return false;
  if (p.L < 4 || p.L > 64) return false;
  if (p.h % kChunkKeys) return false;
  FwdPlan f;
  return plan_forward(p, &f);
}

// sized for the padded image of the tensor-memory variant (L rounded up to a multiple of 4 rows per key)
size_t cimg_bytes(const skv_problem& p) { return align256((size_t)p.h * ((p.L + 3) / 4 * 4) * p.r * sizeof(__half)); }

size_t fwd_scratch_bytes(const skv_problem& p) {
  FwdPlan f;
  if (!plan_forward(p, &f)) return 0;
  return 256 + cimg_bytes(p) + align256((size_t)f.splits * (p.N > 0 ? p.N : 1) * p.r * sizeof(float));
}

// Largest magnitude of C into the scratch header, then the scaled f16 image.
int launch_pack_c(const LaunchCtx& c, const void* C, uint32_t* hdr, void* img, int LP) {
  if (cudaMemsetAsync(hdr, 0, 256, c.stream) != cudaSuccess) return SKV_ERR_LAUNCH;
  const int64_t crows = (int64_t)c.p.h * c.p.L;
  const unsigned agrid = (unsigned)((crows * c.p.r + 2047) / 2048 < 296 ? (crows * c.p.r + 2047) / 2048 : 296);
  tc_amax_kernel<<<agrid, 256, 0, c.stream>>>((const __nv_bfloat16*)C, c.p.r, crows, c.p.r, hdr + kAmaxC);
  const size_t pieces = (size_t)c.p.h * LP * (c.p.r / 8);
  const unsigned grid = (unsigned)((pieces + 255) / 256 < 2048 ? (pieces + 255) / 256 : 2048);
  tc_pack_c_kernel<<<grid, 256, 0, c.stream>>>((const __nv_bfloat16*)C, (__half*)img, c.p.h, c.p.L, LP, c.p.r, hdr);
  note_launches(2);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_LAUNCH;
}

int forward(const LaunchCtx& c, const void* z, int64_t zs, const void* C, void* act_out, int64_t as,
            void* delta_out, int64_t ds, void* scratch, size_t scratch_bytes) {
  const skv_problem& p = c.p;
  FwdPlan f;
  if (!plan_forward(p, &f)) return SKV_ERR_UNSUPPORTED;
  if (scratch_bytes < fwd_scratch_bytes(p)) return SKV_ERR_SCRATCH;
  uint32_t* hdr = reinterpret_cast<uint32_t*>(scratch);                 // 256-byte header: max|C|
  __half* img = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(scratch) + 256);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + 256 + cimg_bytes(p));
  const int LR = (p.L + 1) & ~1;
  if (int e = launch_pack_c(c, C, hdr, img, f.ta ? (((p.L + 1) / 2 + 1) & ~1) * 2 : LR)) return e;

  FwdParams P;
  P.z = (const __nv_bfloat16*)z;
  P.zs = zs;
  P.act_out = (__nv_bfloat16*)act_out;
  P.as = as;
  P.cimg = img;
  P.partial = partial;
  P.N = p.N;
  P.h = p.h;
  P.L = p.L;
  P.r = p.r;
  P.LR = LR;
  P.g = c.g;
  P.act = p.activation;
  P.chunks_total = p.h / kChunkKeys;
  P.chunks_per_split = f.chunks_per_split;
  P.status = c.status;
  P.cstages = f.cstages;
  P.wait_cycles = wait_cycle_limit();
  P.skip_copy = debug_skip_copy() == 1;
  // A: Phi tile, K-major; core matrices of 8 tokens x 8 k: 128 B apart along tokens, 2048 B along k
  P.a_lbo = 2048;
  P.a_sbo = 128;
  // B: code-table chunk, N(=channel)-major; core matrices 128 B apart along channels, r/8*128 B along k
  P.b_lbo = (uint32_t)(p.r / 8) * 128u;
  P.b_sbo = 128;

  const int64_t tiles = (p.N + 128 * f.groups - 1) / (128 * f.groups);
  dim3 grid((unsigned)tiles, (unsigned)f.splits);
  cudaError_t err = cudaErrorInvalidValue;
  if (f.ta) {
    const unsigned threads = 160 * f.groups + 32;
    const int hl = (p.L + 1) / 2;
#define SKV_TA_LAUNCH(G_, HL_, ACT_)                                                                                 \
  {                                                                                                                  \
    err = cudaFuncSetAttribute(tc_forward_ta_kernel<G_, HL_, ACT_, kStagedPerHalf>,                     \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)f.smem);                            \
    if (err == cudaSuccess)                                                                                          \
      tc_forward_ta_kernel<G_, HL_, ACT_, kStagedPerHalf><<<grid, threads, f.smem, c.stream>>>(P);      \
  }
#define SKV_TA_CASE(G_, HL_)                                                                                         \
  if (f.groups == G_ && hl == HL_) {                                                                                 \
    if (p.activation == SKV_ACT_RELU_SQ) SKV_TA_LAUNCH(G_, HL_, SKV_ACT_RELU_SQ)                                     \
    else if (p.activation == SKV_ACT_GELU) SKV_TA_LAUNCH(G_, HL_, SKV_ACT_GELU)                                      \
    else SKV_TA_LAUNCH(G_, HL_, SKV_ACT_IDENTITY)                                                                    \
  }
    SKV_TA_CASE(1, 8) SKV_TA_CASE(2, 8) SKV_TA_CASE(3, 8) SKV_TA_CASE(4, 8)
    SKV_TA_CASE(1, 11) SKV_TA_CASE(2, 11) SKV_TA_CASE(3, 11) SKV_TA_CASE(4, 11)
    SKV_TA_CASE(1, 12) SKV_TA_CASE(2, 12) SKV_TA_CASE(3, 12) SKV_TA_CASE(4, 12)
    SKV_TA_CASE(1, 16) SKV_TA_CASE(2, 16) SKV_TA_CASE(3, 16)
    SKV_TA_CASE(1, 21) SKV_TA_CASE(2, 21)
#undef SKV_TA_LAUNCH
#undef SKV_TA_CASE
  } else if (f.groups == 2) {
    err = cudaFuncSetAttribute(tc_forward_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)f.smem);
    if (err == cudaSuccess) tc_forward_kernel<2><<<grid, 128 * 2 + 64, f.smem, c.stream>>>(P);
  } else {
    err = cudaFuncSetAttribute(tc_forward_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)f.smem);
    if (err == cudaSuccess) tc_forward_kernel<1><<<grid, 128 + 64, f.smem, c.stream>>>(P);
  }
  note_launches(1);
  if (err != cudaSuccess || cudaGetLastError() != cudaSuccess) { cudaGetLastError(); return SKV_ERR_LAUNCH; }

  const int64_t total = p.N * p.r;
  const unsigned fgrid = (unsigned)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
  if (p.delta_f32)
    tc_finalize_kernel<float><<<fgrid, 256, 0, c.stream>>>(partial, f.splits, p.N, p.r, p.lambda_scale, hdr,
                                                           (float*)delta_out, ds);
  else
    tc_finalize_kernel<__nv_bfloat16><<<fgrid, 256, 0, c.stream>>>(partial, f.splits, p.N, p.r, p.lambda_scale, hdr,
                                                                   (__nv_bfloat16*)delta_out, ds);
  note_launches(1);
  return cudaGetLastError() == cudaSuccess ? SKV_OK : SKV_ERR_LAUNCH;
}

}  // namespace tc
}  // namespace skv
