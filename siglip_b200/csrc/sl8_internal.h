// sl8_internal.h -- what the translation units of libsiglip_fp8.so share: the handle, the error helpers and the
// device guard.  Not installed; the public interface is include/siglip_fp8.h.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

#include "../../include/siglip_fp8.h"
#include "sl8_variants.h"

#define SL8_API extern "C" __attribute__((visibility("default")))

typedef CUresult (*sl8_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Staging owned by the handle for the *_host entry points.
struct Sl8HostPipe {
    static const int SLOTS = 3;
    cudaStream_t stream[SLOTS] = {nullptr, nullptr, nullptr};
    cudaEvent_t consts_ready = nullptr;
    void* d_a[SLOTS] = {nullptr, nullptr, nullptr};
    void* d_r[SLOTS] = {nullptr, nullptr, nullptr};
    void* d_d[SLOTS] = {nullptr, nullptr, nullptr};
    void* d_h[SLOTS] = {nullptr, nullptr, nullptr};   // hidden activations of the FC1 -> FC2 chain (never leave the GPU)
    size_t a_bytes = 0, r_bytes = 0, d_bytes = 0, h_bytes = 0;
    void* d_b = nullptr;      size_t b_bytes = 0;
    void* d_bias = nullptr;   size_t bias_bytes = 0;
    void* d_b2 = nullptr;     size_t b2_bytes = 0;     // second weight matrix and bias of the chain
    void* d_bias2 = nullptr;  size_t bias2_bytes = 0;
    void* d_table = nullptr;  size_t table_bytes = 0;
    float* d_scales = nullptr;   // scale_a, scale_b, out_scale (chain: scale_a, scale_w1, hidden_scale, scale_w2)
    float* h_scales = nullptr;   // pinned twin
    bool ready = false;
};

// Tensor maps of recent calls, keyed by everything that goes into one: a layer called again on the same buffers
// (every step of a model) skips the four driver encodes, which cost more host time than the launch itself.
struct Sl8MapCacheEntry {
    int dt = -1, promo = 0, swizzle = 0;
    const void* base = nullptr;
    unsigned long long inner = 0, outer = 0, pitch = 0;
    unsigned box_inner = 0, box_outer = 0;
    CUtensorMap map;
};

struct sl8_context {
    static constexpr int kMapCache = 32;
    Sl8MapCacheEntry map_cache[kMapCache];
    int map_cache_next = 0;
    int device = 0;
    int sm_count = 0;
    uint32_t* d_status = nullptr;       // 4 words
    long long* d_prof = nullptr;        // tracing buffer, PROF_SLOTS per CTA, or null
    int prof_blocks = 0;
    bool test_drop_b = false;           // SL8_TEST_DROP_B=1: test aid, one operand copy is never issued so that a bounded wait expires
    bool single_acc = false;            // SL8_SINGLE_ACC=1: measurement aid, one accumulator (no MMA / epilogue overlap)
    bool trace_coarse = false;          // sl8_trace_enable(h, 2): per-role totals only, untimed code paths
    int last_grid = 0;
    sl8_encode_tiled_fn encode = nullptr;
    int forced_variant = -1;
    int max_clusters_override = 0;      // SL8_MAX_CLUSTERS: measurement aid, caps the persistent grid
    unsigned wait_budget_us = 2000000;
    bool smem_attr_set[SL8_NUM_VARIANTS][sl8::K_COUNT] = {};
    int max_clusters[SL8_NUM_VARIANTS][sl8::K_COUNT] = {};
    std::mutex mu;          // the handle's state during one launch (map cache, attributes, error text)
    std::mutex pipe_mu;     // the host-operand pipeline during one *_host call (taken before mu)
    std::string err;
    Sl8HostPipe pipe;
};

// Records the message (in the handle, or per thread when there is none) and returns `code`.  Defined in sl8_api.cu.
int sl8_fail(sl8_handle_t h, int code, const std::string& msg);
int sl8_fail_cuda(sl8_handle_t h, cudaError_t e, const char* what);

inline bool sl8_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Makes the handle's device current for the duration of a call and puts the caller's back.
struct Sl8DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit Sl8DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~Sl8DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};
