/*
 * sl8_oracle.c -- CPU restatement of the reference's three fused FP8 GEMM layers.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with
 * (tests, the smoke check and the bench's CPU-baseline leg).  Nothing in the product
 * library links, loads or calls it.
 *
 * Parity pin: the closed-form known answers of the reference's own self-validation
 * (A = 0x3C everywhere, B rows alternating 0x3C / 0x38, bias[c] = c + 1,
 * pos[r, c] = 3 (r + 1), residual[r, c] = bf16((r % 128) / 4 + c / 8);
 * patch_embed.cu:121-145,273-306, fc1_gelu.cu:67-85,200-225, fc2.cu:59-66,88-116,231-259)
 * are reproduced bit for bit by tests/test_oracle_golden.py.
 *
 * What is restated (reference file:line):
 *   GEMM            D[m,n] = sum_k A[m,k] * B[n,k], e4m3 x e4m3 -> FP32 accumulate
 *                   kernel_body.cuh:539-545,561-562,586-617 (tile walk, operand
 *                   coordinates, tcgen05.mma kind::f8f6f4 with F32 accumulator
 *                   kernel_common.cuh:111,213-245)
 *   patch-embed     bf16x2(acc) + bf16x2(table[m % SEQ_LEN, n]) in the bf16 domain
 *                   patch_embed.cu:44-58 ; table = bf16(bias + pos) patch_embed.cu:79-98 ;
 *                   row -> period row kernel_body.cuh:71
 *   FC1             gelu_fwd(acc + bias) with tanhf, then cvt.rn.bf16  fc1_gelu.cu:16-19,25-44
 *   FC2             (acc + bias) + float(residual), then cvt.rn.bf16   fc2.cu:19-54
 *   output rounding cvt.rn.bf16x2.f32 (round to nearest even)          kernel_common.cuh:325-345
 *
 * Defined here because the reference has no counterpart (its kernels take raw codes):
 *   acc_scaled = (scale_a * scale_b) * acc          per-tensor dequantisation
 *   e4m3 output = sat_rne(g * (1.0f / out_scale))   FC1 -> FC2 chain
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -fopenmp -shared).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <immintrin.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define SL8O_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ scalar codecs */

/* e4m3 (OCP FP8 E4M3FN): 1 sign, 4 exponent (bias 7), 3 mantissa; no infinity;
 * 0x7F / 0xFF are NaN; largest finite 448 = 0x7E. */
static float e4m3_decode_one(uint8_t c) {
    int s = c >> 7, e = (c >> 3) & 0xF, m = c & 7;
    float v;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);              /* subnormal: m * 2^-9 */
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return s ? -v : v;
}

static float g_e4m3_lut[256];
static int g_lut_ready = 0;
static void lut_init(void) {
    if (g_lut_ready) return;
    for (int i = 0; i < 256; i++) g_e4m3_lut[i] = e4m3_decode_one((uint8_t)i);
    g_lut_ready = 1;
}

SL8O_API float sl8o_e4m3_to_f32(uint8_t c) { lut_init(); return g_e4m3_lut[c]; }

/* Round-to-nearest-even with saturation to +-448 (the behaviour of
 * cvt.rn.satfinite.e4m3x2.f32); NaN -> 0x7F. */
SL8O_API uint8_t sl8o_f32_to_e4m3(float x) {
    if (isnan(x)) return 0x7F;
    uint8_t s = signbit(x) ? 0x80 : 0;
    float a = fabsf(x);
    if (a >= 448.0f) return s | 0x7E;
    if (a < ldexpf(1.0f, -6)) {                        /* subnormal range, step 2^-9 */
        float q = a * 512.0f;                         /* exact (power of two) */
        float r = rintf(q);                           /* default rounding mode = RNE */
        int m = (int)r;                               /* 0..8 ; 8 -> smallest normal */
        if (m >= 8) return s | 0x08;
        return s | (uint8_t)m;
    }
    int e;
    float f = frexpf(a, &e);                           /* a = f * 2^e, f in [0.5,1) */
    float q = f * 16.0f;                               /* in [8,16): 1.mmm * 8 */
    float r = rintf(q);
    int mi = (int)r;
    int E = e - 1;                                     /* unbiased exponent of 1.mmm */
    if (mi == 16) { mi = 8; E += 1; }
    int be = E + 7;
    if (be > 15 || (be == 15 && (mi - 8) == 7)) return s | 0x7E;   /* would be NaN / overflow */
    return s | (uint8_t)((be << 3) | (mi - 8));
}

SL8O_API float sl8o_bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f;
}

/* cvt.rn.bf16.f32 */
SL8O_API uint16_t sl8o_f32_to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;            /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* Round a double to bf16 once (RNE).  Used for add.rn.bf16x2, whose result is the exact
 * sum of two bf16 values rounded once; the exact sum of two bf16 values whose exponents
 * differ by less than 45 fits a double, and beyond that the small operand cannot move
 * the result. */
static uint16_t f64_to_bf16(double d) {
    if (isnan(d)) return 0x7FFF;
    if (d == 0.0 || isinf(d) || fabs(d) < 0x1p-126 || fabs(d) >= 0x1p127)
        return sl8o_f32_to_bf16((float)d);              /* zero, inf, subnormal or near overflow */
    int e;
    double f = frexp(d, &e);                            /* d = f * 2^e, |f| in [0.5, 1) */
    double r = rint(f * 256.0);                         /* 8 significant bits, ties to even */
    float out = (float)ldexp(r, e - 8);                 /* exact: at most 8 significant bits */
    uint32_t u; memcpy(&u, &out, 4);
    return (uint16_t)(u >> 16);
}

/* add.rn.bf16x2 on one lane (patch_embed.cu:51-58). */
SL8O_API uint16_t sl8o_bf16_add(uint16_t a, uint16_t b) {
    return f64_to_bf16((double)sl8o_bf16_to_f32(a) + (double)sl8o_bf16_to_f32(b));
}

/* gelu_fwd, fc1_gelu.cu:16-19. */
SL8O_API float sl8o_gelu_tanh(float x) {
    const float k = 0.7978845608f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

SL8O_API int sl8o_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

SL8O_API void sl8o_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ bulk codecs */

SL8O_API void sl8o_quantize_e4m3(const float* x, int64_t n, float inv_scale, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = sl8o_f32_to_e4m3(x[i] * inv_scale);
}

SL8O_API void sl8o_dequantize_e4m3(const uint8_t* c, int64_t n, float* out) {
    lut_init();
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = g_e4m3_lut[c[i]];
}

/* ------------------------------------------------------------------ GEMM */

typedef float v8f __attribute__((vector_size(32)));
/* acc += a * b on eight lanes as one fused multiply-add.  The product of two e4m3 values has at most eight significant
 * bits, so it is exact in FP32 and the fused form rounds exactly as a separate multiply and add would: the instruction
 * is chosen for speed (this GEMM is also the timed CPU baseline), not for its rounding. */
#define FMA8(acc, a, b) ((acc) = (v8f)_mm256_fmadd_ps((__m256)(a), (__m256)(b), (__m256)(acc)))

static inline float hsum8(v8f v) {
    return ((v[0] + v[4]) + (v[1] + v[5])) + ((v[2] + v[6]) + (v[3] + v[7]));
}

/* Dequantise `rows` rows of an e4m3 matrix into floats with a pitch that is a multiple
 * of 8 (zero padded) so the dot products below need no K tail. */
static float* dequant_rows(const uint8_t* P, int64_t ld, int64_t rows, int K, int Kp) {
    float* F = (float*)aligned_alloc(64, (size_t)rows * Kp * sizeof(float));
    if (!F) return NULL;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const uint8_t* src = P + r * ld;
        float* dst = F + r * Kp;
        for (int k = 0; k < K; k++) dst[k] = g_e4m3_lut[src[k]];
        for (int k = K; k < Kp; k++) dst[k] = 0.0f;
    }
    return F;
}

/* acc[m*ldacc + n] = sum_k float(A[m,k]) * float(B[n,k]), FP32 accumulate.
 * 4 x 2 register tile of dot products, eight partial sums each; blocked so a panel of A
 * and a panel of B stay in the per-core cache.  Returns 0, or -1 if memory ran out. */
SL8O_API int sl8o_gemm_fp8_f32(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb,
                               int64_t M, int N, int K, float* acc, int64_t ldacc) {
    lut_init();
    const int Kp = (K + 7) & ~7;
    float* Af = dequant_rows(A, lda, M, K, Kp);
    float* Bf = dequant_rows(B, ldb, N, K, Kp);
    if (!Af || !Bf) { free(Af); free(Bf); return -1; }
    const int MB = 48, NB = 64;
    const int64_t mblocks = (M + MB - 1) / MB;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t mb = 0; mb < mblocks; mb++) {
        const int64_t m0 = mb * MB, m1 = (m0 + MB < M) ? m0 + MB : M;
        for (int n0 = 0; n0 < N; n0 += NB) {
            const int n1 = (n0 + NB < N) ? n0 + NB : N;
            int64_t m = m0;
            for (; m + 4 <= m1; m += 4) {
                const float *a0 = Af + (m + 0) * Kp, *a1 = Af + (m + 1) * Kp,
                            *a2 = Af + (m + 2) * Kp, *a3 = Af + (m + 3) * Kp;
                int n = n0;
                for (; n + 2 <= n1; n += 2) {
                    const float *b0 = Bf + (int64_t)(n + 0) * Kp, *b1 = Bf + (int64_t)(n + 1) * Kp;
                    v8f c00 = {0}, c01 = {0}, c10 = {0}, c11 = {0}, c20 = {0}, c21 = {0}, c30 = {0}, c31 = {0};
                    for (int k = 0; k < Kp; k += 8) {
                        v8f vb0 = *(const v8f*)(b0 + k), vb1 = *(const v8f*)(b1 + k);
                        v8f va = *(const v8f*)(a0 + k); FMA8(c00, va, vb0); FMA8(c01, va, vb1);
                        va = *(const v8f*)(a1 + k);     FMA8(c10, va, vb0); FMA8(c11, va, vb1);
                        va = *(const v8f*)(a2 + k);     FMA8(c20, va, vb0); FMA8(c21, va, vb1);
                        va = *(const v8f*)(a3 + k);     FMA8(c30, va, vb0); FMA8(c31, va, vb1);
                    }
                    float* o = acc + m * ldacc + n;
                    o[0] = hsum8(c00); o[1] = hsum8(c01); o += ldacc;
                    o[0] = hsum8(c10); o[1] = hsum8(c11); o += ldacc;
                    o[0] = hsum8(c20); o[1] = hsum8(c21); o += ldacc;
                    o[0] = hsum8(c30); o[1] = hsum8(c31);
                }
                for (; n < n1; n++) {
                    const float* b0 = Bf + (int64_t)n * Kp;
                    v8f c0 = {0}, c1 = {0}, c2 = {0}, c3 = {0};
                    for (int k = 0; k < Kp; k += 8) {
                        v8f vb = *(const v8f*)(b0 + k);
                        FMA8(c0, *(const v8f*)(a0 + k), vb); FMA8(c1, *(const v8f*)(a1 + k), vb);
                        FMA8(c2, *(const v8f*)(a2 + k), vb); FMA8(c3, *(const v8f*)(a3 + k), vb);
                    }
                    acc[(m + 0) * ldacc + n] = hsum8(c0); acc[(m + 1) * ldacc + n] = hsum8(c1);
                    acc[(m + 2) * ldacc + n] = hsum8(c2); acc[(m + 3) * ldacc + n] = hsum8(c3);
                }
            }
            for (; m < m1; m++) {
                const float* a0 = Af + m * Kp;
                for (int n = n0; n < n1; n++) {
                    const float* b0 = Bf + (int64_t)n * Kp;
                    v8f c0 = {0};
                    for (int k = 0; k < Kp; k += 8) FMA8(c0, *(const v8f*)(a0 + k), *(const v8f*)(b0 + k));
                    acc[m * ldacc + n] = hsum8(c0);
                }
            }
        }
    }
    free(Af); free(Bf);
    return 0;
}

/* ------------------------------------------------------------------ the three layers
 * Argument meaning is that of include/siglip_fp8.h with host pointers and the scales
 * passed by value.  `flags`: 1 = bias is fp32, 2 = patch-embed adds in fp32. */

enum { F_BIAS_F32 = 1, F_PE_F32_ADD = 2 };

static inline float bias_at(const void* bias, int n, unsigned flags) {
    if (!bias) return 0.0f;
    if (flags & F_BIAS_F32) return ((const float*)bias)[n];
    return sl8o_bf16_to_f32(((const uint16_t*)bias)[n]);
}

/* Rows are processed in slabs so the FP32 accumulator scratch stays small. */
#define SLAB 4096

SL8O_API int sl8o_patch_embed(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb,
                              float scale_a, float scale_b,
                              const uint16_t* table, int64_t ld_table, int period, int row_phase,
                              uint16_t* D, int64_t ldd, int64_t M, int N, int K, unsigned flags) {
    const float s = scale_a * scale_b;
    float* acc = (float*)malloc((size_t)SLAB * N * sizeof(float));
    if (!acc) return -1;
    for (int64_t r0 = 0; r0 < M; r0 += SLAB) {
        const int64_t rows = (r0 + SLAB < M) ? SLAB : M - r0;
        if (sl8o_gemm_fp8_f32(A + r0 * lda, lda, B, ldb, rows, N, K, acc, N)) { free(acc); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < rows; i++) {
            const int64_t m = r0 + i;
            const uint16_t* trow = table + ((m + row_phase) % period) * ld_table;   /* kernel_body.cuh:71 */
            for (int n = 0; n < N; n++) {
                const float v = acc[i * N + n] * s;
                if (flags & F_PE_F32_ADD)
                    D[m * ldd + n] = sl8o_f32_to_bf16(v + sl8o_bf16_to_f32(trow[n]));
                else                                                                /* patch_embed.cu:51-58 */
                    D[m * ldd + n] = sl8o_bf16_add(sl8o_f32_to_bf16(v), trow[n]);
            }
        }
    }
    free(acc);
    return 0;
}

/* out_dtype 0: D is bf16 (uint16_t); 1: D is e4m3 (uint8_t).  ldd in output elements. */
SL8O_API int sl8o_fc1_gelu(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb,
                           float scale_a, float scale_b, const void* bias,
                           void* D, int64_t ldd, int out_dtype, float out_scale,
                           int64_t M, int N, int K, unsigned flags) {
    const float s = scale_a * scale_b;
    const float inv_out = 1.0f / out_scale;
    float* acc = (float*)malloc((size_t)SLAB * N * sizeof(float));
    if (!acc) return -1;
    for (int64_t r0 = 0; r0 < M; r0 += SLAB) {
        const int64_t rows = (r0 + SLAB < M) ? SLAB : M - r0;
        if (sl8o_gemm_fp8_f32(A + r0 * lda, lda, B, ldb, rows, N, K, acc, N)) { free(acc); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < rows; i++) {
            const int64_t m = r0 + i;
            for (int n = 0; n < N; n++) {
                const float x = fmaf(acc[i * N + n], s, bias_at(bias, n, flags));    /* one rounding, as the kernel's FMA */
                const float g = (flags & 4u) ? x : sl8o_gelu_tanh(x);   /* fc1_gelu.cu:16-19; flag 4: no activation */
                if (out_dtype == 0) ((uint16_t*)D)[m * ldd + n] = sl8o_f32_to_bf16(g);
                else ((uint8_t*)D)[m * ldd + n] = sl8o_f32_to_e4m3(g * inv_out);
            }
        }
    }
    free(acc);
    return 0;
}

SL8O_API int sl8o_fc2_residual(const uint8_t* A, int64_t lda, const uint8_t* B, int64_t ldb,
                               float scale_a, float scale_b, const void* bias,
                               const uint16_t* residual, int64_t ldr,
                               uint16_t* D, int64_t ldd, int64_t M, int N, int K, unsigned flags) {
    const float s = scale_a * scale_b;
    float* acc = (float*)malloc((size_t)SLAB * N * sizeof(float));
    if (!acc) return -1;
    for (int64_t r0 = 0; r0 < M; r0 += SLAB) {
        const int64_t rows = (r0 + SLAB < M) ? SLAB : M - r0;
        if (sl8o_gemm_fp8_f32(A + r0 * lda, lda, B, ldb, rows, N, K, acc, N)) { free(acc); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < rows; i++) {
            const int64_t m = r0 + i;
            for (int n = 0; n < N; n++) {
                float t = fmaf(acc[i * N + n], s, bias_at(bias, n, flags));          /* fc2.cu:27-30; one rounding, as the kernel's FMA */
                t = t + sl8o_bf16_to_f32(residual[m * ldr + n]);                    /* fc2.cu:31-46 */
                D[m * ldd + n] = sl8o_f32_to_bf16(t);                               /* fc2.cu:47-50 */
            }
        }
    }
    free(acc);
    return 0;
}

/* bf16(bias[c] + pos[r, c]) as a row-major [period, N] table: the arithmetic of
 * precompute_combined (patch_embed.cu:79-98) without its 32x32 blocking. */
SL8O_API void sl8o_combine_bias_pos(const float* bias, const float* pos, int period, int N, uint16_t* table) {
    for (int r = 0; r < period; r++)
        for (int c = 0; c < N; c++)
            table[(int64_t)r * N + c] = sl8o_f32_to_bf16(bias[c] + pos[(int64_t)r * N + c]);
}

/* ---- producer-side steps (test infrastructure like the rest of this file) -------------------------------
 * Patch unfold + quantisation: the reference describes the patch embedding as "Conv2d as GEMM"
 * (docs/architecture.md:11-12) and feeds its GEMM ready-made rows; the row/column order below is the
 * flattening of a Conv2d weight [N, C, P, P] applied to non-overlapping patches in raster order. */
SL8O_API int sl8o_patchify_quantize(const float* pixels, int images, int C, int H, int W, int P, float scale,
                                    uint8_t* A, int64_t lda, int row_bytes) {
    const int gh = H / P, gw = W / P, K = C * P * P;
    const float inv = 1.0f / scale;
    if (lda < K || row_bytes < K || row_bytes > lda) return -1;
    for (int img = 0; img < images; img++)
        for (int gy = 0; gy < gh; gy++)
            for (int gx = 0; gx < gw; gx++) {
                uint8_t* row = A + (((int64_t)img * gh + gy) * gw + gx) * lda;
                for (int c = 0; c < C; c++)
                    for (int py = 0; py < P; py++)
                        for (int px = 0; px < P; px++) {
                            const float v = pixels[(((int64_t)img * C + c) * H + (gy * P + py)) * W + gx * P + px];
                            row[c * P * P + py * P + px] = sl8o_f32_to_e4m3(v * inv);
                        }
                for (int k = K; k < row_bytes; k++) row[k] = 0;
            }
    return 0;
}

SL8O_API float sl8o_amax(const float* x, int64_t rows, int cols, int64_t ld) {
    float m = 0.0f;
    for (int64_t r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) {
            const float a = fabsf(x[r * ld + c]);
            if (a > m) m = a;
        }
    return m;
}

SL8O_API int sl8o_quantize_rows_e4m3(const float* x, int64_t rows, int cols, int64_t ld, float scale, uint8_t* out, int64_t ld_out) {
    const float inv = 1.0f / scale;
    for (int64_t r = 0; r < rows; r++)
        for (int c = 0; c < cols; c++) out[r * ld_out + c] = sl8o_f32_to_e4m3(x[r * ld + c] * inv);
    return 0;
}

/* LayerNorm -> quantise (the reference lists the fusion as unstarted, docs/architecture.md:92-101): statistics in
 * double, the affine map and the scaling in float as the device does them. */
SL8O_API int sl8o_layernorm_quantize(const float* x, int64_t rows, int cols, int64_t ld, const float* gamma,
                                     const float* beta, float eps, float scale, uint8_t* out, int64_t ld_out) {
    const float inv = 1.0f / scale;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const float* row = x + r * ld;
        double sum = 0.0;
        for (int c = 0; c < cols; c++) sum += row[c];
        const double mean = sum / cols;
        double sq = 0.0;
        for (int c = 0; c < cols; c++) sq += (row[c] - mean) * (row[c] - mean);
        const float rstd = (float)(1.0 / sqrt(sq / cols + (double)eps));
        const float meanf = (float)mean;
        for (int c = 0; c < cols; c++) {
            const float g = gamma ? gamma[c] : 1.0f, b = beta ? beta[c] : 0.0f;
            out[r * ld_out + c] = sl8o_f32_to_e4m3(fmaf((row[c] - meanf) * rstd, g, b) * inv);
        }
    }
    return 0;
}
