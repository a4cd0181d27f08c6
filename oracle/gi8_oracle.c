/*
 * CPU oracle for the INT8 GEMM path.  TEST INFRASTRUCTURE ONLY: this file is the checker that
 * the CUDA kernels are compared against (and the timed CPU baseline); nothing in the shipped
 * library links, imports or falls back to it.
 *
 * It restates, in plain C, the arithmetic contract of the reference operator
 *   gemm_int8.matmul(x, y, alpha) -> bf16 (x @ y.T) * alpha      (gemm_int8/__init__.py:28-37)
 * whose device arithmetic is
 *   - int8 x int8 products accumulated in int32               (csrc/kernels/gemm.cu:33-37, 46-58)
 *   - epilogue LinearCombination<bf16, 8, int32, float> with {alpha, beta = 0}:
 *       out = bf16_rne( fp32_rn(acc) * alpha )                (csrc/kernels/gemm.cu:59-63, 96)
 *   - x is [M,K] row-major, y is [N,K] row-major ("column-major K x N")
 *                                                              (csrc/kernels/gemm.cu:42-44, 76-83)
 * and whose own test pins the result to  x.bfloat16() @ x.bfloat16().t()  (test.py:8,15).
 *
 * The MMA itself lives in NVIDIA/cutlass (git submodule, not vendored in the reference tree, pin
 * unknown).  Its int8 tensor-op default saturates the int32 accumulator; |acc| <= 128*128*K cannot
 * reach 2^31 for K < 131072, so this oracle refuses larger K instead of modelling saturation.
 *
 * The row/column-scaled and blockwise-dequantised variants have NO counterpart in the reference
 * ("parity unpinned" by the reference): their semantics are fixed here, as the definition the CUDA
 * kernels must reproduce bit for bit:
 *   scaled   : out[m,n] = bf16_rne( fp32(acc[m,n]) * (sx[m] * sw[n]) )        product of scales first
 *   blockwise: acc = 0; for kb = 0 .. ceil(K/128)-1 ascending:
 *                 t   = sa[m,kb] * sw[n/128,kb]            (fp32, round to nearest)
 *                 acc = fmaf( fp32(P[m,n,kb]), t, acc )    (P = exact int32 dot over the K block)
 *              out[m,n] = bf16_rne(acc)
 *
 * Threading: rows are split over plain pthreads (gi8o_set_num_threads; default = online cores).
 * Build: see oracle/Makefile (gcc -O3 -ffp-contract=off -shared -fPIC -pthread).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <pthread.h>
#include <stdlib.h>
#include <unistd.h>

#define GI8O_OK 0
#define GI8O_BAD_ARG 1

#define KBLOCK 128

#if defined(__x86_64__) && defined(__GNUC__) && !defined(GI8O_NO_CLONES)
#define GI8O_CLONES __attribute__((target_clones("arch=skylake-avx512", "avx2", "default")))
#else
#define GI8O_CLONES
#endif

/* fp32 -> bf16 bits, round to nearest even; NaN stays NaN (quiet). */
static inline uint16_t bf16_rne(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* Exact int32 dot product of two int8 vectors of length k. */
GI8O_CLONES
static int32_t dot_i8(const int8_t *a, const int8_t *b, int64_t k)
{
    int32_t s = 0;
    for (int64_t i = 0; i < k; ++i) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

static int check_dims(int64_t M, int64_t N, int64_t K)
{
    if (M < 0 || N < 0 || K < 0) return GI8O_BAD_ARG;
    if (K >= 131072) return GI8O_BAD_ARG; /* saturation not modelled */
    return GI8O_OK;
}

/* ---- row-parallel driver over pthreads ------------------------------------------------------ */

static int g_threads = 0; /* 0 = number of online cores */

int gi8o_num_threads(void)
{
    if (g_threads > 0) return g_threads;
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

void gi8o_set_num_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*row_fn)(int64_t r0, int64_t r1, void *ctx);

struct job {
    row_fn fn;
    void *ctx;
    int64_t r0, r1;
};

static void *job_main(void *p)
{
    struct job *j = (struct job *)p;
    j->fn(j->r0, j->r1, j->ctx);
    return NULL;
}

/* Calls fn over [0, rows) split into contiguous chunks, one per thread. */
static void parallel_rows(int64_t rows, row_fn fn, void *ctx)
{
    int nt = gi8o_num_threads();
    if (nt > rows) nt = (int)(rows > 0 ? rows : 1);
    if (nt <= 1) {
        fn(0, rows, ctx);
        return;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
    struct job *jobs = (struct job *)malloc(sizeof(struct job) * (size_t)nt);
    int64_t chunk = (rows + nt - 1) / nt;
    int started = 0;
    for (int t = 0; t < nt; ++t) {
        int64_t r0 = t * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
        if (r0 >= r1) break;
        jobs[t].fn = fn, jobs[t].ctx = ctx, jobs[t].r0 = r0, jobs[t].r1 = r1;
        if (pthread_create(&th[t], NULL, job_main, &jobs[t]) != 0) {
            fn(r0, r1, ctx); /* could not spawn: do the chunk here */
            th[t] = 0;
            jobs[t].fn = NULL;
        }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t)
        if (jobs[t].fn) pthread_join(th[t], NULL);
    free(th);
    free(jobs);
}

struct gemm_ctx {
    const int8_t *x, *y;
    const float *s0, *s1;
    int64_t ld0, ld1;
    void *out;
    float *acc_f32;
    int64_t M, N, K;
    float alpha;
};

/* acc[m,n] = sum_k x[m,k] * y[n,k], exact int32. */
static void rows_i32(int64_t r0, int64_t r1, void *p)
{
    struct gemm_ctx *c = (struct gemm_ctx *)p;
    int32_t *acc = (int32_t *)c->out;
    for (int64_t m = r0; m < r1; ++m)
        for (int64_t n = 0; n < c->N; ++n) acc[m * c->N + n] = dot_i8(c->x + m * c->K, c->y + n * c->K, c->K);
}

int gi8o_matmul_i32(const int8_t *x, const int8_t *y, int32_t *acc, int64_t M, int64_t N, int64_t K)
{
    if (check_dims(M, N, K)) return GI8O_BAD_ARG;
    struct gemm_ctx c = {x, y, NULL, NULL, 0, 0, acc, NULL, M, N, K, 1.0f};
    parallel_rows(M, rows_i32, &c);
    return GI8O_OK;
}

/* out = bf16_rne(fp32_rn(acc) * alpha): gemm.cu:59-63,96 restated. */
static void rows_alpha(int64_t r0, int64_t r1, void *p)
{
    struct gemm_ctx *c = (struct gemm_ctx *)p;
    uint16_t *out = (uint16_t *)c->out;
    for (int64_t m = r0; m < r1; ++m)
        for (int64_t n = 0; n < c->N; ++n) {
            float a = (float)dot_i8(c->x + m * c->K, c->y + n * c->K, c->K);
            out[m * c->N + n] = bf16_rne(a * c->alpha);
        }
}

int gi8o_matmul(const int8_t *x, const int8_t *y, uint16_t *out, int64_t M, int64_t N, int64_t K, float alpha)
{
    if (check_dims(M, N, K)) return GI8O_BAD_ARG;
    struct gemm_ctx c = {x, y, NULL, NULL, 0, 0, out, NULL, M, N, K, alpha};
    parallel_rows(M, rows_alpha, &c);
    return GI8O_OK;
}

/* Per-token (sx[M]) times per-output-channel (sw[N]) scales; the two scales are multiplied first. */
static void rows_scaled(int64_t r0, int64_t r1, void *p)
{
    struct gemm_ctx *c = (struct gemm_ctx *)p;
    uint16_t *out = (uint16_t *)c->out;
    for (int64_t m = r0; m < r1; ++m)
        for (int64_t n = 0; n < c->N; ++n) {
            float a = (float)dot_i8(c->x + m * c->K, c->y + n * c->K, c->K);
            float t = c->s0[m] * c->s1[n];
            out[m * c->N + n] = bf16_rne(a * t);
        }
}

int gi8o_matmul_scaled(const int8_t *x, const int8_t *y, const float *sx, const float *sw, uint16_t *out,
                       int64_t M, int64_t N, int64_t K)
{
    if (check_dims(M, N, K)) return GI8O_BAD_ARG;
    struct gemm_ctx c = {x, y, sx, sw, 0, 0, out, NULL, M, N, K, 1.0f};
    parallel_rows(M, rows_scaled, &c);
    return GI8O_OK;
}

/*
 * Blockwise dequantised GEMM.  sa is [M, ceil(K/128)] with row stride ld_sa (floats); sw is
 * [ceil(N/128), ceil(K/128)] with row stride ld_sw.  If acc_f32 is non-NULL the fp32 accumulator
 * before the bf16 cast is also written there.
 */
static void rows_blockwise(int64_t r0, int64_t r1, void *p)
{
    struct gemm_ctx *c = (struct gemm_ctx *)p;
    uint16_t *out = (uint16_t *)c->out;
    const int64_t K = c->K, N = c->N, KB = (K + KBLOCK - 1) / KBLOCK;
    for (int64_t m = r0; m < r1; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int64_t kb = 0; kb < KB; ++kb) {
                int64_t k0 = kb * KBLOCK;
                int64_t kl = (K - k0 < KBLOCK) ? (K - k0) : KBLOCK;
                float pf = (float)dot_i8(c->x + m * K + k0, c->y + n * K + k0, kl);
                float t = c->s0[m * c->ld0 + kb] * c->s1[(n / KBLOCK) * c->ld1 + kb];
                acc = fmaf(pf, t, acc);
            }
            if (c->acc_f32) c->acc_f32[m * N + n] = acc;
            out[m * N + n] = bf16_rne(acc);
        }
}

int gi8o_matmul_blockwise(const int8_t *x, const int8_t *y, const float *sa, int64_t ld_sa, const float *sw,
                          int64_t ld_sw, uint16_t *out, float *acc_f32, int64_t M, int64_t N, int64_t K)
{
    if (check_dims(M, N, K)) return GI8O_BAD_ARG;
    const int64_t KB = (K + KBLOCK - 1) / KBLOCK;
    if (ld_sa < KB || ld_sw < KB) return GI8O_BAD_ARG;
    struct gemm_ctx c = {x, y, sa, sw, ld_sa, ld_sw, out, acc_f32, M, N, K, 1.0f};
    parallel_rows(M, rows_blockwise, &c);
    return GI8O_OK;
}

/*
 * Symmetric int8 quantisation of a row-major fp32 matrix in blocks of (rb x cb):
 *   s = amax/127 (s = 1 when the block is all zero), q = clamp(rint(v / s), -127, 127).
 * rint() rounds half to even under the default rounding mode.  scales is
 * [ceil(R/rb), ceil(C/cb)] row-major.  Used for the synthetic workloads (per-token-per-128-K
 * activation blocks rb=1, cb=128; per-128x128 weight blocks; per-row scales rb=1, cb=C).
 */
/* Normalised Walsh-Hadamard rotation along each row in blocks of H elements (H a power of two dividing C):
 * in-place butterflies, strides 1, 2, 4, ... ascending, (a, b) -> (a + b, a - b) in fp32, then one multiplication
 * by fp32(H^-1/2).  The reference names the rotation as its use case (README.md:10) and has no code for it; this
 * restates gemm_int8_b200/quant.py:hadamard_rotate.  out may alias in.
 */
int gi8o_hadamard_rotate(const float *in, float *out, int64_t R, int64_t C, int64_t H)
{
    if (R < 0 || C < 0 || H <= 0 || (H & (H - 1)) || C % H) return GI8O_BAD_ARG;
    const float norm = (float)pow((double)H, -0.5);
    for (int64_t r = 0; r < R; ++r)
        for (int64_t b = 0; b < C; b += H) {
            float *y = out + r * C + b;
            if (out != in) memcpy(y, in + r * C + b, sizeof(float) * (size_t)H);
            for (int64_t h = 1; h < H; h <<= 1)
                for (int64_t i = 0; i < H; i += 2 * h)
                    for (int64_t j = i; j < i + h; ++j) {
                        const float x0 = y[j], x1 = y[j + h];
                        y[j] = x0 + x1;
                        y[j + h] = x0 - x1;
                    }
            for (int64_t j = 0; j < H; ++j) y[j] *= norm;
        }
    return GI8O_OK;
}

int gi8o_quantize_blocks(const float *v, int8_t *q, float *scales, int64_t R, int64_t C, int64_t rb, int64_t cb)
{
    if (R < 0 || C < 0 || rb <= 0 || cb <= 0) return GI8O_BAD_ARG;
    const int64_t nrb = (R + rb - 1) / rb, ncb = (C + cb - 1) / cb;
    for (int64_t br = 0; br < nrb; ++br)
        for (int64_t bc = 0; bc < ncb; ++bc) {
            int64_t r1 = (br + 1) * rb < R ? (br + 1) * rb : R;
            int64_t c1 = (bc + 1) * cb < C ? (bc + 1) * cb : C;
            float amax = 0.0f;
            for (int64_t r = br * rb; r < r1; ++r)
                for (int64_t c = bc * cb; c < c1; ++c) {
                    float a = fabsf(v[r * C + c]);
                    if (a > amax) amax = a;
                }
            float s = amax > 0.0f ? amax / 127.0f : 1.0f;
            scales[br * ncb + bc] = s;
            for (int64_t r = br * rb; r < r1; ++r)
                for (int64_t c = bc * cb; c < c1; ++c) {
                    float t = rintf(v[r * C + c] / s);
                    if (t > 127.0f) t = 127.0f;
                    if (t < -127.0f) t = -127.0f;
                    q[r * C + c] = (int8_t)t;
                }
        }
    return GI8O_OK;
}
