// Blackwell (sm_100a) building blocks of the tensor-core kernels: mbarriers with bounded waits,
// TMA bulk copies, tensor-memory allocation, tcgen05 MMA issue / commit / load and the shared-memory
// matrix descriptors of the un-swizzled canonical layouts.
#pragma once

#include "skv_common.cuh"

namespace skv {
namespace tc {

// Status bits a kernel ORs into the caller's status word when a bounded wait runs out.
constexpr int32_t kStatusTimeoutFwd = 0x1;
constexpr int32_t kStatusTimeoutDz = 0x2;
constexpr int32_t kStatusTimeoutDc = 0x4;
constexpr int32_t kStatusTimeoutBwd = 0x8;

// A wait gives up after this many clock cycles unless the host set another limit (about two
// seconds at 2 GHz).  The limit travels in the kernel parameters so that a test can make a wait
// run out within a millisecond.
constexpr long long kDefaultWaitCycles = 4000000000LL;

// Test hooks, set through skv_debug_set (host side, read at launch time).
long long wait_cycle_limit();        // current limit of every bounded wait
int debug_skip_copy();               // 1: the forward's loader leaves out its first code-table copy;
                                     // 2: the read-out GEMM's loader leaves out its first stage
int fused_backward_roles();          // 0: two kernels (default); 3: dz and dC as one kernel where its plan fits
                                     // (1 / 2: that kernel with only its dz / only its dC role, for timing)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for the whole warp: every lane has finished (and fenced) its own writes; after the
// warp-level sync lane 0 arrives for all 32.  A barrier fed this way counts warps, not threads:
// 128 per-thread arrivals on one shared-memory word are 128 serialised atomics on the path between
// a producer's last write and the MMA thread's first instruction.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait with a suspend-time hint: the thread may sleep up to `ns` nanoseconds and is woken when
// the phase completes, so a waiting warp does not compete for issue slots with the working ones.
#ifndef SKV_WAIT_HINT_NS
#define SKV_WAIT_HINT_NS 2000
#endif
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)SKV_WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while; a thread that polls
// several barriers in turn uses this form).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// What a bounded wait needs: `abort` is a CTA-wide flag in shared memory (once any wait of the
// CTA has run out, every later wait returns at once, so the kernel always drains, with invalid
// results and `code` recorded in the caller's status word, instead of hanging).
struct WaitCtx {
  volatile int* abort;
  int32_t* status;
  int32_t code;
  long long limit;
};

__device__ __forceinline__ void wait_give_up(const WaitCtx& w) {
  *w.abort = 1;
  if (w.status) atomicOr(w.status, w.code);
}

// Returns true when the CTA is draining (this wait ran out, or it saw the abort flag while it
// spun); the fast path, a phase that is already complete, reads nothing but the barrier.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w) {
  if (mbar_try_wait(bar, parity)) return false;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait_sleep(bar, parity)) {
    if ((++spins & 15) == 0) {
      if (*w.abort) return true;
      if (clock64() - t0 > w.limit) {
        wait_give_up(w);
        return true;
      }
    }
  }
  return false;
}

// Wait that ignores the abort flag: used once at the end of a kernel for the barrier that the last
// tcgen05.commit arrives on, so that tensor memory is not freed (and the CTA does not exit) while
// MMAs issued before a time-out are still running.  They finish by themselves, so this returns.
__device__ __forceinline__ void mbar_wait_drain(uint64_t* bar, uint32_t parity, long long limit) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > limit) return;
  }
}

// Generic-proxy writes to shared memory made visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// One contiguous TMA bulk copy global -> shared of this CTA; completion is counted on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Tensor memory: one warp allocates `cols` columns (power of two >= 32) and later frees them.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], both operands 16-bit, float32 accumulate; issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with the two descriptors given as 32-bit halves, so that an issue loop only has to
// advance the low words (start address field) by a constant per K step.
__device__ __forceinline__ void umma_f16_split(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Halves of an un-swizzled descriptor (see smem_desc): low word = start address and K stride,
// high word = M/N stride and the sm_100 version bit.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo) {
  return ((addr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint32_t desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3FFFu) | (1u << 14); }

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (lane = row of A,
// each 32-bit column holds two consecutive K elements), B from shared memory.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on `bar` when every MMA this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 16 consecutive float32 columns of this warp's 32 lanes (lane = row) into registers.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of an un-swizzled canonical tile: 8 x 16-byte core matrices,
// `lbo` = byte stride between core matrices along K, `sbo` = byte stride along M/N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of sm_100
  return d;                 // layout type 0 (no swizzle), base offset 0
}

// Instruction descriptor for kind::f16: float32 accumulate, A/B element formats (0 = f16, 1 = bf16),
// operand majors (0 = K-major, 1 = MN-major), tile M x N.
__host__ __device__ constexpr uint32_t instr_desc(int a_fmt, int b_fmt, int a_mn_major, int b_mn_major, int M, int N) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// Range scaling of the f16 operand images.  f16 has a 5-bit exponent: values below 6e-5 lose
// precision and below 3e-8 vanish, which a freshly initialised (near-zero) code table or a small
// upstream gradient would hit.  Each image is therefore multiplied by a power of two chosen from
// the largest magnitude of its source (max * scale lies in [2^12, 2^13); the transformed table's
// second differences then stay below 2^15), and the float32 results are multiplied by the exact
// inverse.
__device__ __forceinline__ void pow2_scales(uint32_t amax_bits, float& scale, float& inv) {
  const int e = (int)((amax_bits >> 23) & 0xff);
  if (e == 0 || e == 255) { scale = 1.0f; inv = 1.0f; return; }
  int se = 127 + 12 - (e - 127);           // biased exponent of 2^(12 - (e-127))
  se = se < 1 ? 1 : (se > 254 ? 254 : se);
  scale = __uint_as_float((uint32_t)se << 23);
  inv = __uint_as_float((uint32_t)(254 - se) << 23);
}
// Words of the 256-byte header at the start of a call's scratch: bit patterns of max|g_delta| and max|C|.
constexpr int kAmaxG = 0, kAmaxC = 8;

namespace {
// Largest magnitude (as a float32 bit pattern, NaN skipped) of a [rows][cols] bf16 array with row stride.
__global__ void tc_amax_kernel(const __nv_bfloat16* __restrict__ a, int64_t stride, int64_t rows, int cols,
                               uint32_t* __restrict__ amax_bits) {
  const int64_t total = rows * cols;
  uint32_t m = 0;
  if (stride == cols && (reinterpret_cast<uintptr_t>(a) & 15) == 0) {
    // contiguous: 16-byte loads; |x| of a bf16 as a float32 bit pattern is its 15 low bits shifted up
    const int64_t n8 = total / 8;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(a) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t lo = (w[q] << 16) & 0x7fff0000u, hi = w[q] & 0x7fff0000u;
        if (lo <= 0x7f800000u) m = max(m, lo);          // NaN patterns lie above infinity: skipped
        if (hi <= 0x7f800000u) m = max(m, hi);
      }
    }
    for (int64_t i = n8 * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
      const float v = fabsf(__bfloat162float(a[i]));
      if (v == v) m = max(m, __float_as_uint(v));
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const float v = fabsf(__bfloat162float(a[(i / cols) * stride + (i % cols)]));
      if (v == v) m = max(m, __float_as_uint(v));
    }
  }
  // one atomic per CTA: thousands of per-warp atomics on one word serialise in L2
  __shared__ uint32_t wmax[32];
  for (int s = 16; s >= 1; s >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < (blockDim.x + 31) / 32 ? wmax[threadIdx.x] : 0u;
    for (int s = 16; s >= 1; s >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
    if (threadIdx.x == 0 && m) atomicMax(amax_bits, m);
  }
}
}  // namespace

// Two float32 -> packed f16x2 (low half = a) as a 32-bit word.
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// ReLU(z)^2 of two packed bf16 values.  The product of two bf16 values is exact in float32, so the
// packed multiply (one rounding to bf16) equals float32 arithmetic followed by a cast.
__device__ __forceinline__ uint32_t relu_sq_bf2(uint32_t w) {
  __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w);
  v = __hmax2(v, __float2bfloat162_rn(0.0f));
  v = __hmul2(v, v);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// ---------------------------------------------------------------------------------------------
// Expanded-basis (Phi) row segment of one (token, key) pair.
//
// A token's Phi row is stored K-major in the un-swizzled canonical layout: 32-bit word w of the
// row (knot columns 2w, 2w+1 as f16x2) lives at byte (w >> 2) * 2048 + (w & 3) * 4 from the
// token's row base, i.e. at word offset w + (w >> 2) * 508.  The three non-zero weights sit at
// columns bin..bin+2 of the key's L columns and always fall into two consecutive words.
// phi_pair returns those two words and their word offsets; `wq` is the word index at which the
// key's segment starts (key-in-chunk * L / 2).
// The weights use B1 = 1 - B0 - B2 (partition of unity), masked by 0 <= u <= G.
// ---------------------------------------------------------------------------------------------
// `kw` is the word distance between consecutive 16-byte chunks of a row minus 4: 508 for tiles of
// 128 token rows (2048 bytes per chunk column), 252 for tiles of 64.
__device__ __forceinline__ void phi_pair(float zz, const GridParams& g, uint32_t wq, uint32_t& x0, uint32_t& x1,
                                         uint32_t& wo0, uint32_t& wo1, uint32_t kw = 508u) {
  const Knot k = knot_of(zz, g);
  const float t = k.tau, omt = 1.0f - t;
  const float hm = k.in_range ? 0.5f : 0.0f;
  const float B0 = (hm * omt) * omt;
  const float B2 = (hm * t) * t;
  const float B1 = fmaf(2.0f, hm, -B0) - B2;          // (m - B0) - B2 with m = 2 * hm, same roundings
  const uint32_t p01 = pack_h2(B0, B1), p2 = pack_h2(B2, 0.0f);
  const uint32_t sh = (k.tbits & 1u) << 4;
  x0 = p01 << sh;
  x1 = __funnelshift_l(p01, p2, sh);
  const uint32_t s0 = wq + ((uint32_t)k.bin >> 1), s1 = s0 + 1u;
  wo0 = s0 + (s0 >> 2) * kw;
  wo1 = s1 + (s1 >> 2) * kw;
}

// phi_pair with the word index s0 of the first word (the second is s0 + 1) instead of offsets.
__device__ __forceinline__ void phi_pair_s(float zz, const GridParams& g, uint32_t wq, uint32_t& x0, uint32_t& x1,
                                           uint32_t& s0) {
  const Knot k = knot_of(zz, g);
  const float t = k.tau, omt = 1.0f - t;
  const float hm = k.in_range ? 0.5f : 0.0f;
  const float B0 = (hm * omt) * omt;
  const float B2 = (hm * t) * t;
  const float B1 = fmaf(2.0f, hm, -B0) - B2;
  const uint32_t p01 = pack_h2(B0, B1), p2 = pack_h2(B2, 0.0f);
  const uint32_t sh = (k.tbits & 1u) << 4;
  x0 = p01 << sh;
  x1 = __funnelshift_l(p01, p2, sh);
  s0 = wq + ((uint32_t)k.bin >> 1);
}

// Knot-dependent part of phi_pair only: the two f16x2 words and the index (bin >> 1) of the first
// one within the key's L/2 words, returned with the bias kWordBias (the callers fold the bias into
// the constants they compare or add it to, which saves an instruction per pair).
constexpr uint32_t kWordBias = kKnotBias >> 1;
__device__ __forceinline__ void phi_pair_words(float zz, const GridParams& g, uint32_t& x0, uint32_t& x1,
                                               uint32_t& wp) {
  const Knot k = knot_of(zz, g);
  const float t = k.tau, omt = 1.0f - t;
  const float hm = k.in_range ? 0.5f : 0.0f;
  const float B0 = (hm * omt) * omt;
  const float B2 = (hm * t) * t;
  const float B1 = fmaf(2.0f, hm, -B0) - B2;          // (m - B0) - B2 with m = 2 * hm, same roundings
  const uint32_t p01 = pack_h2(B0, B1), p2 = pack_h2(B2, 0.0f);
  const uint32_t sh = (k.tbits & 1u) << 4;
  x0 = p01 << sh;
  x1 = __funnelshift_l(p01, p2, sh);
  wp = k.tbits >> 1;
}

// phi_pair_words for the two keys held in one packed bf16 word (low half = first key), with the
// float32 arithmetic issued as two-wide instructions (add / sub / mul / fma .f32x2 of sm_100: each half
// is the same IEEE operation with the same rounding as the scalar instruction, so every result is bit
// for bit that of phi_pair_words).
__device__ __forceinline__ unsigned long long f2_pack(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ void phi_pair_words2(uint32_t zw, const GridParams& g, uint32_t (&x0)[2], uint32_t (&x1)[2],
                                                uint32_t (&wp)[2]) {
  unsigned long long v, u2, t2, tau2, omt2, b0, b2, b1;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(f2_pack(bf_lo(zw), bf_hi(zw))), "l"(f2_pack(g.lo, g.lo)));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(u2) : "l"(v), "l"(f2_pack(g.scale, g.scale)), "l"(0ull));
  float ua, ub;
  f2_unpack(u2, ua, ub);
  const float hma = __float_as_uint(ua) <= __float_as_uint(g.Gf) ? 0.5f : 0.0f;
  const float hmb = __float_as_uint(ub) <= __float_as_uint(g.Gf) ? 0.5f : 0.0f;
  const unsigned long long uc2 = f2_pack(fminf(fmaxf(ua, 0.0f), g.Gm1f), fminf(fmaxf(ub, 0.0f), g.Gm1f));
  const unsigned long long big2 = f2_pack(8388608.0f, 8388608.0f), hm2 = f2_pack(hma, hmb);
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(t2) : "l"(uc2), "l"(big2));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(t2), "l"(big2));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(tau2) : "l"(uc2), "l"(v));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(omt2) : "l"(f2_pack(1.0f, 1.0f)), "l"(tau2));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(hm2), "l"(omt2));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(b0) : "l"(v), "l"(omt2));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(v) : "l"(hm2), "l"(tau2));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(b2) : "l"(v), "l"(tau2));
  asm("add.rn.f32x2 %0, %1, %1;" : "=l"(v) : "l"(hm2));                                    // 2 * hm, exact
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(b0), "l"(f2_pack(-1.0f, -1.0f)), "l"(v));  // 2 hm - B0, one rounding
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(b1) : "l"(v), "l"(b2));
  float ta, tb, B0a, B0b, B1a, B1b, B2a, B2b;
  f2_unpack(t2, ta, tb);
  f2_unpack(b0, B0a, B0b);
  f2_unpack(b1, B1a, B1b);
  f2_unpack(b2, B2a, B2b);
  const uint32_t tba = __float_as_uint(ta), tbb = __float_as_uint(tb);
  const uint32_t p01a = pack_h2(B0a, B1a), p2a = pack_h2(B2a, 0.0f);
  const uint32_t p01b = pack_h2(B0b, B1b), p2b = pack_h2(B2b, 0.0f);
  const uint32_t sha = (tba & 1u) << 4, shb = (tbb & 1u) << 4;
  x0[0] = p01a << sha;
  x1[0] = __funnelshift_l(p01a, p2a, sha);
  wp[0] = tba >> 1;
  x0[1] = p01b << shb;
  x1[1] = __funnelshift_l(p01b, p2b, shb);
  wp[1] = tbb >> 1;
}

// Store N consecutive 32-bit columns of this thread's tensor-memory lane (lane = 32 * (warp % 4) + lane id).
template <int N> __device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t* w);
template <> __device__ __forceinline__ void tmem_st<1>(uint32_t taddr, const uint32_t* w) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(w[0]) : "memory");
}
template <> __device__ __forceinline__ void tmem_st<2>(uint32_t taddr, const uint32_t* w) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(w[0]), "r"(w[1]) : "memory");
}
template <> __device__ __forceinline__ void tmem_st<4>(uint32_t taddr, const uint32_t* w) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(w[0]), "r"(w[1]),
               "r"(w[2]), "r"(w[3])
               : "memory");
}
template <> __device__ __forceinline__ void tmem_st<8>(uint32_t taddr, const uint32_t* w) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(w[0]),
               "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
template <> __device__ __forceinline__ void tmem_st<16>(uint32_t taddr, const uint32_t* w) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};" ::"r"(taddr),
      "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "r"(w[8]), "r"(w[9]),
      "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15])
      : "memory");
}
template <> __device__ __forceinline__ void tmem_st<32>(uint32_t taddr, const uint32_t* w) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "r"(w[8]), "r"(w[9]),
      "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]), "r"(w[16]), "r"(w[17]), "r"(w[18]),
      "r"(w[19]), "r"(w[20]), "r"(w[21]), "r"(w[22]), "r"(w[23]), "r"(w[24]), "r"(w[25]), "r"(w[26]), "r"(w[27]),
      "r"(w[28]), "r"(w[29]), "r"(w[30]), "r"(w[31])
      : "memory");
}
// HL (< 64) consecutive columns as the binary decomposition of HL into x16/x8/x4/x2/x1 stores.
template <int HL> __device__ __forceinline__ void tmem_st_words(uint32_t taddr, const uint32_t* w) {
  int o = 0;
  if constexpr ((HL & 32) != 0) { tmem_st<32>(taddr, w); o += 32; }
  if constexpr ((HL & 16) != 0) { tmem_st<16>(taddr + o, w + o); o += 16; }
  if constexpr ((HL & 8) != 0) { tmem_st<8>(taddr + o, w + o); o += 8; }
  if constexpr ((HL & 4) != 0) { tmem_st<4>(taddr + o, w + o); o += 4; }
  if constexpr ((HL & 2) != 0) { tmem_st<2>(taddr + o, w + o); o += 2; }
  if constexpr ((HL & 1) != 0) { tmem_st<1>(taddr + o, w + o); o += 1; }
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

}  // namespace tc
}  // namespace skv
