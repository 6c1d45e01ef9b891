/*
 * splinekv_b200 -- C ABI of the B200 (sm_100a) implementation of the RL-Spline-KV
 * feature operator:
 *
 *   forward    f = [ phi(z) ; lambda * delta ],   delta[n,:] = sum_j sum_{k<3} B_k(z[n,j]) * C[j, bin(z[n,j]) + k, :]
 *   backward   dz = g_a * phi'(z) + lambda * scale * sum_k B_k'(z) <g_delta, C[j, bin+k, :]>
 *              dC = lambda * Phi(z)^T g_delta
 *
 * z is [N, h] (tokens x keys), C is [h, L, r] with L = G + 2 knot rows (G + 1 for the linear
 * spline, skv_problem.spline_order), outputs are in
 * the dtype of z.  Every entry point takes plain device pointers, sizes and a CUDA stream
 * handle (cudaStream_t passed as void*); none of them allocates, frees, synchronises or
 * throws.  They enqueue work on the given stream and return 0 or a negative SKV_ERR_* code.
 *
 * Each declaration names the interface of the reference project it replaces
 * (paths inside that project).
 */
#ifndef SPLINEKV_B200_H
#define SPLINEKV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKV_ABI_VERSION 4

enum skv_error {
  SKV_OK = 0,
  SKV_ERR_NULL = -1,        /* a required pointer is NULL */
  SKV_ERR_SHAPE = -2,       /* N, h, L, r out of range, or L < 4 */
  SKV_ERR_UNSUPPORTED = -3, /* dtype / activation / impl not supported for this shape */
  SKV_ERR_ALIGN = -4,       /* pointer or stride alignment the chosen kernel needs is not met */
  SKV_ERR_SCRATCH = -5,     /* scratch buffer missing or smaller than skv_scratch_bytes() */
  SKV_ERR_DEVICE = -6,      /* current device is not compute capability 10.x */
  SKV_ERR_LAUNCH = -7,      /* a kernel launch failed (cudaGetLastError) */
  SKV_ERR_NOALLOC_LIMIT = -8 /* problem needs more than SKV_NOALLOC_SCRATCH_BYTES of scratch */
};

enum skv_dtype { SKV_BF16 = 0, SKV_F32 = 1 };
enum skv_activation { SKV_ACT_RELU_SQ = 0, SKV_ACT_IDENTITY = 1, SKV_ACT_GELU = 2 };
/* SKV_IMPL_AUTO picks the tcgen05 kernels when the shape is eligible (bf16, r a multiple of 16
 * up to 128, L up to 64, h a multiple of 8, 16-byte aligned rows) and the CUDA-core kernels
 * otherwise.  The CUDA-core kernels are the float32 tier and a correctness fallback, tens of
 * times slower at production sizes: skv_resolve_impl tells which family a problem gets. */
enum skv_impl { SKV_IMPL_AUTO = 0, SKV_IMPL_SIMT = 1, SKV_IMPL_TCGEN05 = 2 };
enum skv_op { SKV_OP_FORWARD = 0, SKV_OP_BACKWARD = 1 };

/* Problem description shared by all entry points.  `scale` is float32(G / (grid_hi - grid_lo))
 * with the division done in double by the caller, as the reference's Python wrappers do
 * (src/sparsespline_ffn/cuda_ext/__init__.py:334-352, 529-555). */
typedef struct skv_problem {
  int64_t N;           /* tokens */
  int32_t h;           /* keys */
  int32_t L;           /* knot rows per key, = G + 2 (G + 1 when spline_order is 1) */
  int32_t r;           /* code dimension */
  float grid_lo;
  float scale;
  float lambda_scale;
  int32_t activation;  /* enum skv_activation */
  int32_t dtype;       /* enum skv_dtype: dtype of z, C, grad_out, f, dz */
  int32_t impl;        /* enum skv_impl */
  int32_t delta_f32;   /* forward only: 1 = write lambda*delta as float32 whatever dtype is (the
                          key-sharded mode sums partial residuals across GPUs in float32) */
  int32_t dz_f32;      /* backward only, tcgen05 kernels: 1 = write dz as float32 (before its rounding
                          to the dtype of z), so that a systematic error of dz can be measured; the
                          dz pointer and stride are then in float32 elements */
  int32_t spline_order; /* 0 or 2: quadratic B-spline, L = G + 2 (the operator of the reference's kernels);
                          1: linear B-spline, L = G + 1, weights 1 - tau and tau at rows bin, bin + 1
                          (_b1_basis_and_bins, src/sparsespline_ffn/rl_spline_kv_reference.py:125-142, which the
                          reference evaluates in PyTorch only); runs on the CUDA-core kernels */
} skv_problem;

/* ABI version of the loaded library (SKV_ABI_VERSION). */
int skv_abi_version(void);

/* Human-readable text for a SKV_ERR_* code. */
const char *skv_error_string(int code);

/* 0 when the current CUDA device can run this library (compute capability 10.x), else SKV_ERR_DEVICE.
 * Replaces the capability gates of the reference loaders (src/sparsespline_ffn/cuda_ext/__init__.py:31-60). */
int skv_device_ok(void);

/* Which kernels SKV_IMPL_AUTO resolves to for this problem: SKV_IMPL_SIMT or SKV_IMPL_TCGEN05
 * (negative SKV_ERR_* when the problem is invalid).  Replaces the eligibility tests of
 * FlashSplineFeature.forward (src/sparsespline_ffn/kernels/flash_spline_feature_autograd.py:64-82). */
int skv_resolve_impl(const skv_problem *p);

/* Bytes of caller-owned scratch that op (enum skv_op) needs for this problem.  The reference
 * kernels allocate theirs internally (src/sparsespline_ffn/cuda_ext/spline_kv_fwd_v11.cu:372-375,
 * src/sparsespline_ffn/cuda_ext/spline_kv_bwd_wgmma_v5.cu:588-598). */
size_t skv_scratch_bytes(const skv_problem *p, int op);

/* Forward.  Replaces spline_kv_fwd_cuda / spline_kv_fwd_v11_cuda
 * (src/sparsespline_ffn/cuda_ext/__init__.py:529-555, src/sparsespline_ffn/cuda_ext/spline_kv_fwd_v11.cu:349-402)
 * and the Triton forward flash_spline_feature_forward
 * (src/sparsespline_ffn/kernels/triton_flash_spline_feature.py:273-369).
 *   z          [N, h], row stride z_stride elements, unit inner stride
 *   C          [h, L, r] contiguous
 *   act_out    [N, h] phi(z), row stride act_stride; NULL for the delta-only operator
 *   delta_out  [N, r] lambda*delta, row stride delta_stride in elements of its own type (for the
 *              feature operator pass &f[0][h] and stride h + r so that both halves land in one
 *              tensor); float32 when p->delta_f32 is set, else the dtype of z
 *   status     optional device int32; a kernel writes a non-zero code there if one of its
 *              bounded waits ran out (results are then invalid) */
int skv_feature_forward(const skv_problem *p, const void *z, int64_t z_stride, const void *C,
                        void *act_out, int64_t act_stride, void *delta_out, int64_t delta_stride,
                        void *scratch, size_t scratch_bytes, int32_t *status, void *stream);

/* Backward.  Replaces spline_kv_bwd_wgmma_cuda(_fused) / spline_kv_bwd_wgmma_v5_cuda
 * (src/sparsespline_ffn/cuda_ext/spline_kv_bwd_wgmma.cu:508-584,
 * src/sparsespline_ffn/cuda_ext/spline_kv_bwd_wgmma_v5.cu:553-621), the Triton backward
 * flash_spline_delta_backward_v3 (src/sparsespline_ffn/kernels/triton_flash_spline_feature.py:1294-1331)
 * and the elementwise tail of FlashSplineFeature.backward
 * (src/sparsespline_ffn/kernels/flash_spline_feature_autograd.py:146-152, 226-242).
 *   g_act    [N, h] gradient of the phi(z) half, row stride gact_stride; NULL for delta-only
 *   g_delta  [N, r] gradient of the lambda*delta half (NOT pre-multiplied by lambda)
 *   dz       [N, h] out, dtype of z; NULL to skip
 *   dC_f32   [h, L, r] float32 out (overwritten, not accumulated); NULL to skip
 *   dC_cast  optional [h, L, r] copy of dC in the dtype of C */
int skv_feature_backward(const skv_problem *p, const void *z, int64_t z_stride, const void *C,
                         const void *g_act, int64_t gact_stride, const void *g_delta, int64_t gdelta_stride,
                         void *dz, int64_t dz_stride, float *dC_f32, void *dC_cast,
                         void *scratch, size_t scratch_bytes, int32_t *status, void *stream);

/* Knot-interval index of every z[n, j] as int32 [N, h] (contiguous), computed by the same device
 * function all kernels use.  Lets a caller check indices bit for bit against
 * _b2_basis_and_bins (src/sparsespline_ffn/rl_spline_kv_reference.py:88-109). */
int skv_knot_index(const skv_problem *p, const void *z, int64_t z_stride, int32_t *bins, void *stream);

/* Feature followed by its read-out projection, without the feature tensor in between:
 *   y[N, d_out] = phi(z) . W_out[:, 0:h]^T + (lambda * delta(z, C)) . W_out[:, h:h+r]^T
 * Replaces spline_kv_fwd_fused_cuda (src/sparsespline_ffn/cuda_ext/spline_kv_fwd.cu:307-417, wrapper
 * src/sparsespline_ffn/cuda_ext/__init__.py:617-647), which writes phi(z) and delta to memory and calls two
 * library GEMMs.  Here delta comes from the feature kernels in their delta-only mode and one tcgen05 GEMM
 * over K = h + r applies phi to the z tile on its way into shared memory; phi(z) and delta are rounded to
 * bf16 before the product and the accumulation is float32, as in the reference.  Forward only, like the
 * reference's entry point.
 *   w_out    [d_out, h + r] bf16, row stride w_stride elements (the layout of torch.nn.Linear.weight)
 *   y        [N, d_out] bf16 out, row stride y_stride
 * Needs dtype bf16, activation relu_sq or identity, h, r, d_out, the three row strides multiples of 8 and
 * 16-byte aligned pointers (else SKV_ERR_UNSUPPORTED / SKV_ERR_ALIGN), N below 2^31 - 256.  Scratch:
 * skv_readout_scratch_bytes(p, d_out) bytes at a 256-byte aligned address (else SKV_ERR_SCRATCH).  A bounded wait of the GEMM that runs out sets bit 0x10 of *status. */
size_t skv_readout_scratch_bytes(const skv_problem *p, int64_t d_out);
int skv_feature_readout_forward(const skv_problem *p, const void *z, int64_t z_stride, const void *C,
                                const void *w_out, int64_t w_stride, int64_t d_out, void *y, int64_t y_stride,
                                void *scratch, size_t scratch_bytes, int32_t *status, void *stream);

/* Forward for callers that cannot allocate device memory (no counterpart in the reference, whose
 * kernels allocate their scratch themselves through the PyTorch allocator).  Same arguments and
 * results as skv_feature_forward minus the scratch pair: the scratch is a fixed array of
 * SKV_NOALLOC_SCRATCH_BYTES inside the library's device image, which every GPU that loads the
 * library holds until the process exits.  It exists for hosts where cudaMalloc is not an option
 * when the operator runs: servers and plugin sandboxes that fix their device memory at
 * start-up, and latency-critical loops that cannot afford an allocation's cost and implicit
 * synchronisation.  This call itself uses no cudaMalloc, cudaFree or allocating library
 * routine.  (Nothing is stated here about recording it into a CUDA graph.)
 *  - A problem whose skv_scratch_bytes(p, SKV_OP_FORWARD) exceeds the array is refused with
 *    SKV_ERR_NOALLOC_LIMIT (at h = 5120, L = 22, r = 32, N = 4096 tokens fit and N = 8192
 *    do not; the need is not monotonic in N because the number of key splits depends on it,
 *    so ask skv_scratch_bytes; use skv_feature_forward with caller-owned scratch beyond the limit).
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call before any stream
 *    capture begins.
 *  - All calls on a device share the one array.  Its contents are whatever the previous call
 *    left; the forward overwrites everything it reads, so nothing needs clearing, but two calls
 *    whose kernels overlap on the GPU (for instance on different streams)
 *    race on it.  Serialise them. */
#define SKV_NOALLOC_SCRATCH_BYTES (16u << 20)
int skv_feature_forward_noalloc(const skv_problem *p, const void *z, int64_t z_stride, const void *C,
                                void *act_out, int64_t act_stride, void *delta_out, int64_t delta_stride,
                                int32_t *status, void *stream);

/* Debug and test settings; no counterpart in the reference (whose kernels wait on their barriers
 * without a limit, src/sparsespline_ffn/cuda_ext/spline_kv_bwd_v6.cu:159-172).  Process-wide, read when a
 * kernel is launched.
 *   SKV_DEBUG_WAIT_CYCLES      limit of every bounded device-side wait, in SM clock cycles
 *                              (default 4e9, about two seconds); a wait that runs out sets a bit
 *                              in the caller's status word and the kernel returns by itself
 *   SKV_DEBUG_SKIP_FIRST_COPY  1: the forward's loader leaves out its first code-table copy, so
 *                              that a wait runs out although nothing is in flight (tests of the
 *                              time-out path); 2: the same for the first stage of the read-out
 *                              GEMM; 0 restores normal operation
 *   SKV_DEBUG_FUSED_BACKWARD   1: run dz and dC as one kernel (dedicated warps per role in one
 *                              CTA) where its plan fits, instead of the two kernels used by
 *                              default; same results, measured no faster (A/B timing, tests) */
enum skv_debug { SKV_DEBUG_WAIT_CYCLES = 0, SKV_DEBUG_SKIP_FIRST_COPY = 1, SKV_DEBUG_FUSED_BACKWARD = 2 };
int skv_debug_set(int what, int64_t value);

/* Number of kernels this library has launched in this process so far (host-side counter).  No
 * counterpart in the reference; benchmarks use the difference around a timed region to report
 * how many of the library's own kernels ran inside it. */
uint64_t skv_kernel_launches(void);

#ifdef __cplusplus
}
#endif
#endif /* SPLINEKV_B200_H */
