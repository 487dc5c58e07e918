// sl8_bench.cu -- per-layer bench host over the C ABI, speaking the reference harness's protocol.
//
// Counterpart of the reference's three bench hosts (patch_embed.cu:104-346, fc1_gelu.cu:52-254,
// fc2.cu:72-289): same constant operands (A = 0x3C, B rows alternating 0x3C / 0x38, bias[c] = c + 1,
// pos[r, c] = 3 (r + 1), residual[r, c] = bf16((r % 128) / 4 + c / 8)), same 2 warm-up + 10 timed launches
// under one event pair, same 32 closed-form spot checks and 1024-sample strided checksum, and the same
// machine-readable line its drivers parse (tools/grid_search.py:153-158, tools/compare_all.py:90-100):
//
//     @@RESULT ms=%.3f tflops=%.2f checksum=%f valid=%d c0=%.1f
//
// plus "Custom kernel: %.3f ms" for tools/stat_test.py:27.  Shapes are run-time here:
//
//     siglip_bench --layer pe|fc1|fc2 [--M rows] [--N n] [--K k] [--period p] [--runs r]
//     siglip_bench --config C1|C2|C3|C4            (the benchmark configurations: layer and shape in one word)
//
// Defaults are the reference's: M = 928256, patch-embed 768 x 768 period 196, FC1 3072 x 768, FC2 768 x 3072.
// A JSON line with the same figures follows the @@RESULT line.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/siglip_fp8.h"

#define CHECK_CUDA(x)                                                                             \
    do {                                                                                          \
        cudaError_t e_ = (x);                                                                     \
        if (e_ != cudaSuccess) {                                                                  \
            fprintf(stderr, "CUDA %s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));      \
            return 1;                                                                             \
        }                                                                                         \
    } while (0)

#define CHECK_SL8(h, x)                                                                           \
    do {                                                                                          \
        int r_ = (x);                                                                             \
        if (r_ != SL8_OK) {                                                                       \
            fprintf(stderr, "sl8 %s:%d: %d %s\n", __FILE__, __LINE__, r_, sl8_last_error_string(h)); \
            return 1;                                                                             \
        }                                                                                         \
    } while (0)

static __global__ void fill_residual(__nv_bfloat16* res, int n, long long total) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx < total) {
        const int col = static_cast<int>(idx % n);
        const long long row = idx / n;
        res[idx] = __float2bfloat16(static_cast<float>(row % 128) * 0.25f + static_cast<float>(col) * 0.125f);
    }
}

static float gelu_host(float x) {   // fc1_gelu.cu:16-19
    const float k = 0.7978845608f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
}

static float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

int main(int argc, char** argv) {
    setbuf(stdout, NULL);
    const char* layer = "pe";
    long long M = 928256;
    int N = -1, K = -1, period = 196, runs = 10;
    for (int i = 1; i < argc; i++) {
        if (!strcmp(argv[i], "--layer") && i + 1 < argc) layer = argv[++i];
        else if (!strcmp(argv[i], "--M") && i + 1 < argc) M = atoll(argv[++i]);
        else if (!strcmp(argv[i], "--N") && i + 1 < argc) N = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--K") && i + 1 < argc) K = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--period") && i + 1 < argc) period = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--runs") && i + 1 < argc) runs = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--config") && i + 1 < argc) {
            const char* c = argv[++i];
            if (!strcmp(c, "C1")) { layer = "pe"; M = 6272; N = 768; K = 768; period = 196; }
            else if (!strcmp(c, "C2")) { layer = "fc1"; M = 46656; N = 4304; K = 1152; }
            else if (!strcmp(c, "C3")) { layer = "fc2"; M = 46656; N = 1152; K = 4304; }
            else if (!strcmp(c, "C4")) { layer = "pe"; M = 186624; N = 1152; K = 588; period = 729; }
            else { fprintf(stderr, "unknown config %s (C1..C4)\n", c); return 2; }
        }
        else {
            fprintf(stderr, "usage: %s [--config C1|C2|C3|C4] [--layer pe|fc1|fc2] [--M rows] [--N n] [--K k] [--period p] [--runs r]\n", argv[0]);
            return 2;
        }
    }
    const int op = !strcmp(layer, "pe") ? SL8_OP_PATCH_EMBED : !strcmp(layer, "fc1") ? SL8_OP_FC1_GELU : !strcmp(layer, "fc2") ? SL8_OP_FC2_RESIDUAL : -1;
    if (op < 0) { fprintf(stderr, "unknown layer %s\n", layer); return 2; }
    if (N < 0) N = op == SL8_OP_FC1_GELU ? 3072 : 768;
    if (K < 0) K = op == SL8_OP_FC2_RESIDUAL ? 3072 : 768;
    const long long lda = (K + 127) / 128 * 128;      // rows start on 128-byte lines

    sl8_handle_t h = NULL;
    if (sl8_create(&h, 0) != SL8_OK) { fprintf(stderr, "sl8_create: %s\n", sl8_last_error_string(NULL)); return 1; }
    sl8_config cfg;
    CHECK_SL8(h, sl8_query_config(h, op, SL8_OUT_BF16, M, N, K, &cfg));
    printf("%s GEMM -- %s, [%lld,%d] x [%d,%d]^T, tile %dx%dx%d, cta_group::%d, %d stages, %d epilogue warps, grid %d\n",
           layer, sl8_version(), M, K, N, K, cfg.tile_m, cfg.tile_n, cfg.tile_k, cfg.cta_group, cfg.stages, cfg.epi_warps, cfg.grid);

    // ---- operands: the reference's constant test vectors (patch_embed.cu:121-145, fc2.cu:59-66)
    uint8_t *d_A, *d_B;
    __nv_bfloat16 *d_C, *d_table = NULL, *d_res = NULL;
    float *d_bias, *d_pos = NULL;
    CHECK_CUDA(cudaMalloc(&d_A, static_cast<size_t>(M) * lda));
    CHECK_CUDA(cudaMalloc(&d_B, static_cast<size_t>(N) * lda));
    CHECK_CUDA(cudaMalloc(&d_bias, static_cast<size_t>(N) * sizeof(float)));
    CHECK_CUDA(cudaMalloc(&d_C, static_cast<size_t>(M) * N * sizeof(__nv_bfloat16)));
    CHECK_CUDA(cudaMemset(d_A, 0x3C, static_cast<size_t>(M) * lda));                     // 1.5
    {
        std::vector<uint8_t> hB(static_cast<size_t>(N) * lda, 0);
        for (int n = 0; n < N; n++) memset(hB.data() + static_cast<size_t>(n) * lda, (n & 1) ? 0x38 : 0x3C, K);   // 1.0 / 1.5
        CHECK_CUDA(cudaMemcpy(d_B, hB.data(), hB.size(), cudaMemcpyHostToDevice));
        std::vector<float> hb(N);
        for (int c = 0; c < N; c++) hb[c] = static_cast<float>(c + 1);
        CHECK_CUDA(cudaMemcpy(d_bias, hb.data(), N * sizeof(float), cudaMemcpyHostToDevice));
    }
    int table_rows = 0;
    if (op == SL8_OP_PATCH_EMBED) {
        std::vector<float> hp(static_cast<size_t>(period) * N);
        for (int r = 0; r < period; r++)
            for (int c = 0; c < N; c++) hp[static_cast<size_t>(r) * N + c] = 3.0f * static_cast<float>(r + 1);
        CHECK_CUDA(cudaMalloc(&d_pos, hp.size() * sizeof(float)));
        CHECK_CUDA(cudaMemcpy(d_pos, hp.data(), hp.size() * sizeof(float), cudaMemcpyHostToDevice));
        table_rows = sl8_padded_table_rows(period);
        CHECK_CUDA(cudaMalloc(&d_table, static_cast<size_t>(table_rows) * N * sizeof(__nv_bfloat16)));
        CHECK_SL8(h, sl8_make_periodic_table(h, d_bias, d_pos, period, N, d_table, N, table_rows, 0));   // precompute_combined
    }
    if (op == SL8_OP_FC2_RESIDUAL) {
        const long long total = M * N;
        CHECK_CUDA(cudaMalloc(&d_res, static_cast<size_t>(total) * sizeof(__nv_bfloat16)));
        fill_residual<<<static_cast<unsigned>((total + 255) / 256), 256>>>(d_res, N, total);
        CHECK_CUDA(cudaGetLastError());
    }
    CHECK_CUDA(cudaDeviceSynchronize());
    printf("  Alloc + init done\n");

    auto launch = [&]() -> int {
        if (op == SL8_OP_PATCH_EMBED)
            return sl8_patch_embed_fp8(h, d_A, lda, d_B, lda, NULL, NULL, d_table, N, period, table_rows, 0, d_C, N, M, N, K, 0, 0);
        if (op == SL8_OP_FC1_GELU)
            return sl8_fc1_gelu_fp8(h, d_A, lda, d_B, lda, NULL, NULL, d_bias, d_C, N, SL8_OUT_BF16, NULL, M, N, K, SL8_FLAG_BIAS_F32, 0);
        return sl8_fc2_residual_fp8(h, d_A, lda, d_B, lda, NULL, NULL, d_bias, d_res, N, d_C, N, M, N, K, SL8_FLAG_BIAS_F32, 0);
    };

    // ---- 2 warm-up + `runs` timed launches under one event pair (patch_embed.cu:213-246)
    for (int i = 0; i < 2; i++) CHECK_SL8(h, launch());
    CHECK_CUDA(cudaDeviceSynchronize());
    cudaEvent_t e0, e1;
    CHECK_CUDA(cudaEventCreate(&e0));
    CHECK_CUDA(cudaEventCreate(&e1));
    CHECK_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < runs; i++) CHECK_SL8(h, launch());
    CHECK_CUDA(cudaEventRecord(e1));
    CHECK_CUDA(cudaEventSynchronize(e1));
    float total_ms = 0;
    CHECK_CUDA(cudaEventElapsedTime(&total_ms, e0, e1));
    const double ms = total_ms / runs;
    unsigned detail[4];
    CHECK_SL8(h, sl8_device_status(h, 0, detail));
    const double tflops = 2.0 * M * N * K / ms / 1e9;
    printf("Custom kernel: %.3f ms  %.2f TFLOPS\n", ms, tflops);

    // ---- validation on the host: 32 spots + checksum (patch_embed.cu:249-306)
    std::vector<__nv_bfloat16> hC(static_cast<size_t>(M) * N);
    CHECK_CUDA(cudaMemcpy(hC.data(), d_C, hC.size() * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost));
    double cksum = 0;
    {
        const long long stride = M * N / 1024;
        for (int i = 0; i < 1024; i++) cksum += std::fabs(static_cast<double>(__bfloat162float(hC[static_cast<size_t>(i) * stride])));
    }
    int errors = 0;
    for (int spot = 0; spot < 32; spot++) {
        const long long row = spot * M / 32;
        const int col = (spot * 47) % N;
        const float gemm = static_cast<float>(K) * 1.5f * ((col & 1) ? 1.0f : 1.5f);
        const float bias = static_cast<float>(col + 1);
        float expect;
        if (op == SL8_OP_PATCH_EMBED) {
            const float comb = bf16_round(bias + 3.0f * static_cast<float>(row % period + 1));
            expect = bf16_round(bf16_round(gemm) + comb);                                   // patch_embed.cu:281-292
        } else if (op == SL8_OP_FC1_GELU) {
            expect = bf16_round(gelu_host(gemm + bias));                                    // fc1_gelu.cu:207-211
        } else {
            const float res = bf16_round(static_cast<float>(row % 128) * 0.25f + static_cast<float>(col) * 0.125f);
            expect = bf16_round(gemm + bias + res);                                         // fc2.cu:239-245
        }
        const float got = __bfloat162float(hC[static_cast<size_t>(row) * N + col]);
        if (got != expect) {
            if (errors < 5) printf("  MISMATCH at (%lld,%d): expected %.1f got %.1f\n", row, col, expect, got);
            errors++;
        }
    }
    const int valid = errors == 0;
    printf("Validation: %d/32 spot checks passed%s\n", 32 - errors, valid ? "" : " -- FAILED");
    printf("Checksum (1024 strided, absolute values): %f\n", cksum);
    // the reference's parsers accept [0-9.] only: a non-negative fixed-notation checksum and |c0|
    printf("@@RESULT ms=%.3f tflops=%.2f checksum=%f valid=%d c0=%.1f\n", ms, tflops, cksum, valid,
           std::fabs(__bfloat162float(hC[0])));
    printf("{\"layer\": \"%s\", \"M\": %lld, \"N\": %d, \"K\": %d, \"ms\": %.4f, \"tflops\": %.2f, \"valid\": %d, \"variant\": %d, "
           "\"runs\": %d, \"operands\": \"reference constants\"}\n", layer, M, N, K, ms, tflops, valid, cfg.variant_id, runs);

    cudaFree(d_A); cudaFree(d_B); cudaFree(d_bias); cudaFree(d_C);
    if (d_pos) cudaFree(d_pos);
    if (d_table) cudaFree(d_table);
    if (d_res) cudaFree(d_res);
    sl8_destroy(h);
    return valid ? 0 : 1;
}
