/*
 * CPU oracle for the RL-Spline-KV feature path, plain C + OpenMP.
 * TEST INFRASTRUCTURE ONLY: the checker that the CUDA kernels are compared
 * against and the timed CPU baseline.  The shipped library never links it.
 *
 * It restates the algorithm of the reference package's PyTorch oracle
 * (paths inside the reference project):
 *   knot interval + B-spline weights  src/sparsespline_ffn/rl_spline_kv_reference.py:88-109
 *   forward delta gather-sum          src/sparsespline_ffn/rl_spline_kv_reference.py:189-203
 *   analytic dC / dz_spline, masks    src/sparsespline_ffn/kernels/flash_spline_feature_backward_ref.py:96-150
 *   base-path gradient, lambda rule   src/sparsespline_ffn/kernels/flash_spline_feature_autograd.py:146-152, 226-242
 *
 * Parity is pinned: tests/test_oracle_golden.py checks this file (through
 * oracle/c_binding.py) against outputs of the reference itself stored under
 * tests/golden/.
 *
 * Inputs are float32 (bf16 tensors are up-cast by the caller, which is exact).
 * The knot index is computed as the reference computes it in float32:
 * u = fl(fl(z - lo) * scale), no fused multiply-add.  Sums over keys and over
 * tokens are accumulated in double.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC spline_kv_oracle.c -o libskv_oracle.so
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int bin;          /* knot interval in [0, G-1] */
    float B[3];       /* forward weights, forward mask applied */
    float dB[3];      /* derivative weights, clamp mask applied */
} skvo_basis;

/* order 2: quadratic B-spline (rl_spline_kv_reference.py:88-109, three weights at rows bin..bin+2);
 * order 1: linear B-spline (_b1_basis_and_bins, rl_spline_kv_reference.py:125-142: weights 1-tau and
 * tau at rows bin, bin+1; the third weight is zero and its row is never read). */
static inline skvo_basis skvo_eval_o(float z, float lo, float scale, int G, int order)
{
    skvo_basis o;
    volatile float d = z - lo;            /* keep the two roundings separate */
    float u = d * scale;
    int in_range = (u >= 0.0f) && (u <= (float)G);
    int clamp_active = (u >= 0.0f) && (u <= (float)(G - 1));
    float uc = u;
    if (!(uc >= 0.0f)) uc = 0.0f;
    if (uc > (float)(G - 1)) uc = (float)(G - 1);
    int b = (int)uc;                       /* uc >= 0: truncation is floor */
    float tau = uc - (float)b;
    if (tau < 0.0f) tau = 0.0f;
    if (tau > 1.0f) tau = 1.0f;
    float omt = 1.0f - tau;
    float m = in_range ? 1.0f : 0.0f;
    float c = clamp_active ? 1.0f : 0.0f;
    o.bin = b;
    if (order == 1) {
        o.B[0] = omt * m;
        o.B[1] = tau * m;
        o.B[2] = 0.0f;
        o.dB[0] = -c;
        o.dB[1] = c;
        o.dB[2] = 0.0f;
        return o;
    }
    o.B[0] = 0.5f * omt * omt * m;
    o.B[1] = 0.5f * (1.0f + 2.0f * tau - 2.0f * tau * tau) * m;
    o.B[2] = 0.5f * tau * tau * m;
    o.dB[0] = -omt * c;
    o.dB[1] = (1.0f - 2.0f * tau) * c;
    o.dB[2] = tau * c;
    return o;
}

static inline skvo_basis skvo_eval(float z, float lo, float scale, int G)
{
    return skvo_eval_o(z, lo, scale, G, 2);
}

int skvo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Number of OpenMP threads the next calls use (a launcher may have exported OMP_NUM_THREADS=1). */
void skvo_set_threads(int n)
{
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* bins[N*h] (int32), row-major; z has row stride zs (elements). */
void skvo_knot_index(const float *z, int64_t zs, int64_t N, int h,
                     float lo, float scale, int G, int32_t *bins)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int j = 0; j < h; ++j)
            bins[n * h + j] = skvo_eval(z[n * zs + j], lo, scale, G).bin;
}

/* phi and phi' of the base path (rl_spline_kv_reference.py:78-85; the gelu of F.gelu is the exact
 * erf form, its derivative Phi(z) + z * pdf(z) is what autograd returns at
 * flash_spline_feature_autograd.py:229-235). */
static double skvo_act(float zz, int act)
{
    if (act == 0) return zz > 0.0f ? (double)zz * (double)zz : 0.0;
    if (act == 2) return 0.5 * (double)zz * (1.0 + erf((double)zz * 0.70710678118654752440));
    return (double)zz;
}
static double skvo_act_grad(float zz, int act)
{
    if (act == 0) return zz > 0.0f ? 2.0 * (double)zz : 0.0;
    if (act == 2) {
        double x = (double)zz;
        return 0.5 * (1.0 + erf(x * 0.70710678118654752440)) + x * exp(-0.5 * x * x) * 0.39894228040143267794;
    }
    return 1.0;
}

/* act: 0 = relu_sq, 1 = identity, 2 = gelu.
 * a[N*h] (may be NULL) receives phi(z); delta[N*r] receives lambda * delta. */
void skvo_forward_o(const float *z, int64_t zs, const float *C, int64_t N, int h, int L, int r,
                    float lo, float scale, float lambda, int act, int order, float *a, float *delta)
{
    int G = L - order;
    int nb = order + 1;                      /* rows with a weight */
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (size_t)r);
#pragma omp for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            for (int c = 0; c < r; ++c) acc[c] = 0.0;
            for (int j = 0; j < h; ++j) {
                float zz = z[n * zs + j];
                if (a) a[n * h + j] = (float)skvo_act(zz, act);
                skvo_basis e = skvo_eval_o(zz, lo, scale, G, order);
                const float *row = C + ((size_t)j * L + e.bin) * r;
                for (int k = 0; k < nb; ++k) {
                    double bk = e.B[k];
                    for (int c = 0; c < r; ++c) acc[c] += bk * row[(size_t)k * r + c];
                }
            }
            for (int c = 0; c < r; ++c) delta[n * r + c] = (float)((double)lambda * acc[c]);
        }
        free(acc);
    }
}

/* Backward of f = [phi(z); lambda*delta].
 *   g_delta[N*r] (row stride gds): gradient w.r.t. the lambda*delta half.
 *   g_a[N*h] (row stride gas) may be NULL (delta-only operator).
 *   dz[N*h] float32 out = g_a*phi'(z) + lambda*dz_spline.
 *   dC[h*L*r] double out = lambda * Phi^T g_delta. */
void skvo_backward_o(const float *z, int64_t zs, const float *C,
                     const float *g_delta, int64_t gds, const float *g_a, int64_t gas,
                     int64_t N, int h, int L, int r, float lo, float scale, float lambda, int act, int order,
                     float *dz, double *dC)
{
    int G = L - order;
    int nb = order + 1;
    /* dz: parallel over tokens */
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float *g = g_delta + n * gds;
        for (int j = 0; j < h; ++j) {
            float zz = z[n * zs + j];
            skvo_basis e = skvo_eval_o(zz, lo, scale, G, order);
            const float *row = C + ((size_t)j * L + e.bin) * r;
            double sum = 0.0;
            for (int k = 0; k < nb; ++k) {
                double sk = 0.0;
                for (int c = 0; c < r; ++c) sk += (double)g[c] * row[(size_t)k * r + c];
                sum += e.dB[k] * sk;
            }
            double v = (double)lambda * (double)scale * sum;
            if (g_a) {
                double dphi = skvo_act_grad(zz, act);
                v += (double)g_a[n * gas + j] * dphi;
            }
            dz[n * h + j] = (float)v;
        }
    }
    /* dC: parallel over keys, every key owns its [L, r] slab */
#pragma omp parallel for schedule(static)
    for (int j = 0; j < h; ++j) {
        double *slab = dC + (size_t)j * L * r;
        memset(slab, 0, sizeof(double) * (size_t)L * r);
        for (int64_t n = 0; n < N; ++n) {
            skvo_basis e = skvo_eval_o(z[n * zs + j], lo, scale, G, order);
            const float *g = g_delta + n * gds;
            double *row = slab + (size_t)e.bin * r;
            for (int k = 0; k < nb; ++k) {
                double bk = e.B[k];
                for (int c = 0; c < r; ++c) row[(size_t)k * r + c] += bk * (double)g[c];
            }
        }
        for (size_t i = 0; i < (size_t)L * r; ++i) slab[i] *= (double)lambda;
    }
}

/* The quadratic spline under the names the first version of this file exported. */
void skvo_forward(const float *z, int64_t zs, const float *C, int64_t N, int h, int L, int r,
                  float lo, float scale, float lambda, int act, float *a, float *delta)
{
    skvo_forward_o(z, zs, C, N, h, L, r, lo, scale, lambda, act, 2, a, delta);
}

void skvo_backward(const float *z, int64_t zs, const float *C,
                   const float *g_delta, int64_t gds, const float *g_a, int64_t gas,
                   int64_t N, int h, int L, int r, float lo, float scale, float lambda, int act,
                   float *dz, double *dC)
{
    skvo_backward_o(z, zs, C, g_delta, gds, g_a, gas, N, h, L, r, lo, scale, lambda, act, 2, dz, dC);
}
