// sl8_api.cu -- the C ABI of libsiglip_fp8.so (include/siglip_fp8.h): handle life cycle,
// argument validation, tensor-map encoding, the dispatch table and the launches.
//
// This file plays the part of the host half of each reference layer's main()
// (patch_embed.cu:104-246, fc1_gelu.cu:52-170, fc2.cu:72-200): it builds the three tensor
// maps, raises the dynamic shared-memory limit and launches the persistent kernel -- for
// run-time shapes, and returning status codes instead of exiting.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/siglip_fp8.h"
#include "sl8_variants.h"
#include "sl8_dispatch_table.h"

#define SL8_API extern "C" __attribute__((visibility("default")))

namespace {

using sl8::KernelParams;
using sl8::VariantEntry;

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

const VariantEntry* variant(int id) {
    switch (id) {
#define SL8_CASE(id_, CG, TN, TK, ST, EW, NB) \
    case id_:                             \
        return sl8_variant_##id_();
        SL8_VARIANT_LIST(SL8_CASE)
#undef SL8_CASE
        default:
            return nullptr;
    }
}

thread_local std::string g_create_error;

// Staging owned by the handle for the *_host entry points.
struct HostPipe {
    static const int SLOTS = 3;
    cudaStream_t stream[SLOTS] = {nullptr, nullptr, nullptr};
    cudaEvent_t consts_ready = nullptr;
    void* d_a[SLOTS] = {nullptr, nullptr, nullptr};
    void* d_r[SLOTS] = {nullptr, nullptr, nullptr};
    void* d_d[SLOTS] = {nullptr, nullptr, nullptr};
    size_t a_bytes = 0, r_bytes = 0, d_bytes = 0;
    void* d_b = nullptr;      size_t b_bytes = 0;
    void* d_bias = nullptr;   size_t bias_bytes = 0;
    void* d_table = nullptr;  size_t table_bytes = 0;
    float* d_scales = nullptr;   // scale_a, scale_b, out_scale
    float* h_scales = nullptr;   // pinned twin
    bool ready = false;
};

}  // namespace

// Tensor maps of recent calls, keyed by everything that goes into one: a layer called again on the same buffers
// (every step of a model) skips the four driver encodes, which cost more host time than the launch itself.
struct MapCacheEntry {
    int dt = -1, promo = 0;
    const void* base = nullptr;
    unsigned long long inner = 0, outer = 0, pitch = 0;
    unsigned box_inner = 0, box_outer = 0;
    CUtensorMap map;
};

struct sl8_context {
    static constexpr int kMapCache = 32;
    MapCacheEntry map_cache[kMapCache];
    int map_cache_next = 0;
    int device = 0;
    int sm_count = 0;
    uint32_t* d_status = nullptr;       // 4 words
    long long* d_prof = nullptr;        // tracing buffer, PROF_SLOTS per CTA, or null
    int prof_blocks = 0;
    int last_grid = 0;
    encode_tiled_fn encode = nullptr;
    int forced_variant = -1;
    int max_clusters_override = 0;      // SL8_MAX_CLUSTERS: measurement aid, caps the persistent grid
    unsigned wait_budget_ms = 2000;
    bool smem_attr_set[SL8_NUM_VARIANTS][sl8::K_COUNT] = {};
    int max_clusters[SL8_NUM_VARIANTS][sl8::K_COUNT] = {};
    std::mutex mu;
    std::string err;
    HostPipe pipe;
};

namespace {

int fail(sl8_handle_t h, int code, const std::string& msg) {
    if (h) h->err = msg;
    else g_create_error = msg;
    return code;
}

int fail_cuda(sl8_handle_t h, cudaError_t e, const char* what) {
    return fail(h, SL8_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// ---- dispatch -------------------------------------------------------------------------
// The table is generated from a sweep on B200 (python -m siglip_b200.sweep); shapes it does not hold fall back
// to rules (one line per rule; the first match wins).
int kernel_slot(int op, int out_dtype) {
    if (op == SL8_OP_PATCH_EMBED) return sl8::K_PE;
    if (op == SL8_OP_FC2_RESIDUAL) return sl8::K_FC2;
    return out_dtype == SL8_OUT_E4M3 ? sl8::K_FC1_E4M3 : sl8::K_FC1_BF16;
}

int pick_variant(int op, int out_dtype, long long M, int N, int K) {
    // A (layer, N, K) the committed sweep covers: the row with the largest m_min <= M decides.
    int swept = -1;
    long long swept_m = -1;
    for (int i = 0; i < kSl8DispatchRows; i++) {
        const Sl8DispatchRow& r = kSl8DispatchTable[i];
        if (r.op == op && r.n == N && r.k == K && r.m_min <= M && r.m_min > swept_m) {
            swept = r.variant;
            swept_m = r.m_min;
        }
    }
    // (the sweep times bf16 outputs; a variant that has no kernel for this output type is passed over)
    if (swept >= 0 && swept < SL8_NUM_VARIANTS && variant(swept) && variant(swept)->kernel[kernel_slot(op, out_dtype)]) return swept;
    // Any other shape: the rules the sweeps suggest.
    const long long tiles256 = ((M + 255) / 256) * ((N + 255) / 256);
    if (tiles256 < 37) {
        // Fewer 256 x 256 tiles than half the CTA pairs (M sweep: M = 729 .. 1458 at the So400m shapes):
        // 128 x 128 tiles on single CTAs give more of the 148 SMs work.
        return 6;
    }
    // A tcgen05.mma of a CTA pair takes about 150 cycles whatever its N (measured for N = 128, 192,
    // 256), so the widest tile does the most work per instruction even where N = 1152 leaves the
    // fifth 256-wide tile half empty.
    if (op == SL8_OP_FC1_GELU) return 2;      // GELU epilogue: two epilogue warps per scheduler
    if (op == SL8_OP_PATCH_EMBED) return 5;   // short K: four staging boxes keep the table loads ahead of the epilogue
    return 1;
}

struct Problem {
    int op;
    int out_dtype;
    const void *A, *B;
    long long lda, ldb;
    const float *scale_a, *scale_b, *out_scale;
    const void* bias;
    const void* side;
    long long ld_side;
    int period, row_phase, table_rows;
    void* D;
    long long ldd;
    long long M;
    int N, K;
    unsigned flags;
};

int validate(sl8_handle_t h, const Problem& q) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!q.A || !q.B || !q.D) return fail(h, SL8_ERR_INVALID_VALUE, "A, B and D must not be NULL");
    if (q.M < 1 || q.N < 1 || q.K < 1) return fail(h, SL8_ERR_INVALID_VALUE, "M, N, K must be positive");
    if (q.M > 0x7FFFFF00ll) return fail(h, SL8_ERR_UNSUPPORTED, "M exceeds 2^31 rows");
    if (q.out_dtype != SL8_OUT_BF16 && q.out_dtype != SL8_OUT_E4M3)
        return fail(h, SL8_ERR_INVALID_VALUE, "unknown out_dtype");
#ifdef SL8_DIAG
    constexpr unsigned kDiagBits = 0xFFFFFF00u;   // measurement builds only: skip-a-part switches
#else
    constexpr unsigned kDiagBits = 0u;
#endif
    if (q.flags & ~(unsigned)(SL8_FLAG_BIAS_F32 | SL8_FLAG_PE_F32_ADD | SL8_FLAG_NO_ACTIVATION | SL8_FLAG_GELU_HW_TANH | kDiagBits))
        return fail(h, SL8_ERR_INVALID_VALUE, "unknown flag bits");
    if ((q.flags & (SL8_FLAG_NO_ACTIVATION | SL8_FLAG_GELU_HW_TANH)) && q.op != SL8_OP_FC1_GELU)
        return fail(h, SL8_ERR_INVALID_VALUE, "SL8_FLAG_NO_ACTIVATION / SL8_FLAG_GELU_HW_TANH belong to the FC1 entry points");
    if ((q.flags & SL8_FLAG_NO_ACTIVATION) && (q.flags & SL8_FLAG_GELU_HW_TANH))
        return fail(h, SL8_ERR_INVALID_VALUE, "SL8_FLAG_NO_ACTIVATION and SL8_FLAG_GELU_HW_TANH exclude each other");
    if (q.N % 16 != 0) return fail(h, SL8_ERR_UNSUPPORTED, "N must be a multiple of 16");
    if (q.lda < q.K || q.ldb < q.K) return fail(h, SL8_ERR_INVALID_VALUE, "lda / ldb smaller than K");
    if (q.ldd < q.N) return fail(h, SL8_ERR_INVALID_VALUE, "ldd smaller than N");
    const int ob = (q.out_dtype == SL8_OUT_BF16) ? 2 : 1;
    if (!aligned16(q.A) || !aligned16(q.B) || !aligned16(q.D)) return fail(h, SL8_ERR_ALIGNMENT, "A, B, D must be 16-byte aligned");
    if (q.lda % 16 || q.ldb % 16) return fail(h, SL8_ERR_ALIGNMENT, "lda and ldb must be multiples of 16 bytes");
    if ((q.ldd * ob) % 16) return fail(h, SL8_ERR_ALIGNMENT, "row pitch of D must be a multiple of 16 bytes");
    if (q.op == SL8_OP_PATCH_EMBED) {
        if (!q.side) return fail(h, SL8_ERR_INVALID_VALUE, "table must not be NULL");
        if (q.period < 1 || q.row_phase < 0) return fail(h, SL8_ERR_INVALID_VALUE, "period must be positive, row_phase non-negative");
        if (q.table_rows < q.period) return fail(h, SL8_ERR_INVALID_VALUE, "table_rows smaller than period");
        if (q.ld_side < q.N) return fail(h, SL8_ERR_INVALID_VALUE, "ld_table smaller than N");
        if (!aligned16(q.side) || (q.ld_side * 2) % 16) return fail(h, SL8_ERR_ALIGNMENT, "table must be 16-byte aligned with a 16-byte pitch");
    }
    if (q.op == SL8_OP_FC2_RESIDUAL) {
        if (!q.side) return fail(h, SL8_ERR_INVALID_VALUE, "residual must not be NULL");
        if (q.ld_side < q.N) return fail(h, SL8_ERR_INVALID_VALUE, "ldr smaller than N");
        if (!aligned16(q.side) || (q.ld_side * 2) % 16) return fail(h, SL8_ERR_ALIGNMENT, "residual must be 16-byte aligned with a 16-byte pitch");
    }
    if (q.bias && !aligned16(q.bias)) return fail(h, SL8_ERR_ALIGNMENT, "bias must be 16-byte aligned");
    if (q.scale_a && (reinterpret_cast<uintptr_t>(q.scale_a) & 3u)) return fail(h, SL8_ERR_ALIGNMENT, "scale pointers must be 4-byte aligned");
    if (q.scale_b && (reinterpret_cast<uintptr_t>(q.scale_b) & 3u)) return fail(h, SL8_ERR_ALIGNMENT, "scale pointers must be 4-byte aligned");
    if (q.out_scale && (reinterpret_cast<uintptr_t>(q.out_scale) & 3u)) return fail(h, SL8_ERR_ALIGNMENT, "scale pointers must be 4-byte aligned");
    return SL8_OK;
}

int encode_2d(sl8_handle_t h, CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
              unsigned long long inner, unsigned long long outer, unsigned long long pitch_bytes, unsigned box_inner,
              unsigned box_outer, CUtensorMapL2promotion promo) {
    for (int i = 0; i < sl8_context::kMapCache; i++) {      // callers hold h->mu
        const MapCacheEntry& c = h->map_cache[i];
        if (c.base == base && c.dt == (int)dt && c.promo == (int)promo && c.inner == inner && c.outer == outer &&
            c.pitch == pitch_bytes && c.box_inner == box_inner && c.box_outer == box_outer) {
            *map = c.map;
            return SL8_OK;
        }
    }
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    CUresult r = h->encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        MapCacheEntry& c = h->map_cache[h->map_cache_next];
        h->map_cache_next = (h->map_cache_next + 1) % sl8_context::kMapCache;
        c.dt = (int)dt; c.promo = (int)promo; c.base = base; c.inner = inner; c.outer = outer; c.pitch = pitch_bytes;
        c.box_inner = box_inner; c.box_outer = box_outer; c.map = *map;
    }
    if (r != CUDA_SUCCESS) {
        char buf[160];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (CUresult %d) dims {%llu,%llu} pitch %llu box {%u,%u}",
                 (int)r, inner, outer, pitch_bytes, box_inner, box_outer);
        return fail(h, SL8_ERR_CUDA, buf);
    }
    return SL8_OK;
}

int grid_for(sl8_handle_t h, const VariantEntry* v, int slot, int num_tiles) {
    int& cached = h->max_clusters[v->id][slot];
    if (cached == 0) {
        int clusters = h->sm_count / v->cg;
        if (v->cg == 2) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(h->sm_count / 2 * 2), 1, 1);
            cfg.blockDim = dim3(static_cast<unsigned>(v->threads), 1, 1);
            cfg.dynamicSmemBytes = static_cast<size_t>(v->smem_bytes[slot]);
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, v->kernel[slot], &cfg) == cudaSuccess && n > 0 && n < clusters) clusters = n;
            else (void)cudaGetLastError();
        }
        cached = clusters > 0 ? clusters : 1;
    }
    int clusters = num_tiles < cached ? num_tiles : cached;
    if (h->max_clusters_override > 0 && clusters > h->max_clusters_override) clusters = h->max_clusters_override;
    return clusters * v->cg;
}

int run(sl8_handle_t h, const Problem& q, cudaStream_t stream) {
    int rc = validate(h, q);
    if (rc != SL8_OK) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");

    int vid = h->forced_variant >= 0 ? h->forced_variant : pick_variant(q.op, q.out_dtype, q.M, q.N, q.K);
    const VariantEntry* v = variant(vid);
    if (!v) return fail(h, SL8_ERR_INVALID_VALUE, "no such kernel variant");
    const int slot = kernel_slot(q.op, q.out_dtype);
    const int ob = (q.out_dtype == SL8_OUT_BF16) ? 2 : 1;
    if (!v->kernel[slot]) return fail(h, SL8_ERR_UNSUPPORTED, "the forced kernel variant does not serve this layer / output type");

    if (!h->smem_attr_set[vid][slot]) {
        cudaError_t e = cudaFuncSetAttribute(v->kernel[slot], cudaFuncAttributeMaxDynamicSharedMemorySize, v->smem_bytes[slot]);
        if (e != cudaSuccess) return fail_cuda(h, e, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
        h->smem_attr_set[vid][slot] = true;
    }

    CUtensorMap map_a, map_b, map_d;
    rc = encode_2d(h, &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.A, (unsigned long long)q.K, (unsigned long long)q.M,
                   (unsigned long long)q.lda, 128, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != SL8_OK) return rc;
    rc = encode_2d(h, &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.B, (unsigned long long)q.K, (unsigned long long)q.N,
                   (unsigned long long)q.ldb, 128, (unsigned)(v->tn / v->cg), CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != SL8_OK) return rc;
    rc = encode_2d(h, &map_d, ob == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, ob, q.D,
                   (unsigned long long)q.N, (unsigned long long)q.M, (unsigned long long)q.ldd * ob,
                   (unsigned)(128 / ob), 32, CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (rc != SL8_OK) return rc;

    // Side data (table [period, N] or residual [M, N], bf16) comes in by TMA as 128-row x 64-column boxes.
    CUtensorMap map_s = map_d;
    if (q.op == SL8_OP_PATCH_EMBED) {
        rc = encode_2d(h, &map_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q.side, (unsigned long long)q.N,
                       (unsigned long long)q.table_rows, (unsigned long long)q.ld_side * 2, 64, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (rc != SL8_OK) return rc;
    } else if (q.op == SL8_OP_FC2_RESIDUAL) {
        rc = encode_2d(h, &map_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q.side, (unsigned long long)q.N,
                       (unsigned long long)q.M, (unsigned long long)q.ld_side * 2, 64, 128, CU_TENSOR_MAP_L2_PROMOTION_NONE);
        if (rc != SL8_OK) return rc;
    }

    KernelParams p;
    memset(&p, 0, sizeof p);
    p.M = q.M;
    p.N = q.N;
    p.K = q.K;
    const int tile_m = 128 * v->cg;
    const long long tiles_m = (q.M + tile_m - 1) / tile_m;
    p.tiles_n = (q.N + v->tn - 1) / v->tn;
    const long long nt = tiles_m * p.tiles_n;
    if (nt > 0x7FFFFFFFll) return fail(h, SL8_ERR_UNSUPPORTED, "too many tiles");
    p.num_tiles = static_cast<int>(nt);
    p.k_blocks = (q.K + v->tk - 1) / v->tk;
    const int k_last = q.K - (p.k_blocks - 1) * v->tk;
    p.last_kblock_mmas = (k_last + 31) / 32;
    p.scale_a = q.scale_a;
    p.scale_b = q.scale_b;
    p.out_scale = q.out_scale;
    p.bias = q.bias;
    p.side = static_cast<const __nv_bfloat16*>(q.side);
    p.ld_side = q.ld_side;
    p.period = q.period > 0 ? q.period : 1;
    p.row_phase = q.row_phase;
    p.table_rows = q.table_rows;
    p.D = q.D;
    p.ldd = q.ldd;
    p.flags = q.flags;
    p.wait_budget_ms = h->wait_budget_ms;
    p.status = h->d_status;
    p.prof = h->d_prof;

    const int grid = grid_for(h, v, slot, p.num_tiles);
    h->last_grid = grid;
    if (h->d_prof && grid > h->prof_blocks) return fail(h, SL8_ERR_INVALID_VALUE, "tracing buffer smaller than the grid");
    cudaError_t e = v->launch[slot](&map_a, &map_b, &map_d, &map_s, &p, grid, stream);
    if (e != cudaSuccess) return fail_cuda(h, e, "kernel launch");
    return SL8_OK;
}

void fill_config(const VariantEntry* v, int slot, int grid, sl8_config* out) {
    out->cta_group = v->cg;
    out->tile_m = 128 * v->cg;
    out->tile_n = v->tn;
    out->tile_k = v->tk;
    out->stages = v->stages;
    out->epi_warps = v->epi_warps;
    out->staging_buffers = v->nbuf;
    out->grid = grid;
    out->smem_bytes = v->smem_bytes[slot];
    out->variant_id = v->id;
}

}  // namespace

// =========================================================================== life cycle

SL8_API const char* sl8_version(void) { return "siglip_fp8 0.1 sm_100a"; }

SL8_API int sl8_create(sl8_handle_t* out, int device) {
    if (!out) return fail(nullptr, SL8_ERR_INVALID_VALUE, "handle pointer is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        (void)cudaGetLastError();
        return fail(nullptr, SL8_ERR_NO_DEVICE, std::string("no CUDA device: ") + cudaGetErrorString(e));
    }
    if (device < 0 || device >= count) return fail(nullptr, SL8_ERR_INVALID_VALUE, "device index out of range");
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail_cuda(nullptr, e, "cudaGetDeviceProperties");
    if (prop.major != 10 || prop.minor != 0) {
        char buf[128];
        snprintf(buf, sizeof buf, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
        return fail(nullptr, SL8_ERR_ARCH, buf);
    }
    DeviceGuard guard(device);
    if (!guard.ok) return fail(nullptr, SL8_ERR_CUDA, "cudaSetDevice failed");

    sl8_context* h = new (std::nothrow) sl8_context();
    if (!h) return fail(nullptr, SL8_ERR_CUDA, "out of host memory");
    h->device = device;
    h->sm_count = prop.multiProcessorCount;

    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
        delete h;
        return fail(nullptr, SL8_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
    }
    h->encode = reinterpret_cast<encode_tiled_fn>(fn);

    e = cudaMalloc(reinterpret_cast<void**>(&h->d_status), 16);
    if (e != cudaSuccess) {
        delete h;
        return fail_cuda(nullptr, e, "cudaMalloc(status block)");
    }
    e = cudaMemset(h->d_status, 0, 16);
    if (e != cudaSuccess) {
        cudaFree(h->d_status);
        delete h;
        return fail_cuda(nullptr, e, "cudaMemset(status block)");
    }
    const char* mc = getenv("SL8_MAX_CLUSTERS");
    if (mc && *mc) h->max_clusters_override = atoi(mc);
    const char* fv = getenv("SL8_FORCE_VARIANT");
    if (fv && *fv) {
        const int id = atoi(fv);
        if (id >= 0 && id < SL8_NUM_VARIANTS) h->forced_variant = id;
    }
    *out = h;
    return SL8_OK;
}

SL8_API int sl8_destroy(sl8_handle_t h) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    {
        DeviceGuard guard(h->device);
        cudaDeviceSynchronize();
        HostPipe& pp = h->pipe;
        for (int i = 0; i < HostPipe::SLOTS; i++) {
            if (pp.d_a[i]) cudaFree(pp.d_a[i]);
            if (pp.d_r[i]) cudaFree(pp.d_r[i]);
            if (pp.d_d[i]) cudaFree(pp.d_d[i]);
            if (pp.stream[i]) cudaStreamDestroy(pp.stream[i]);
        }
        if (pp.consts_ready) cudaEventDestroy(pp.consts_ready);
        if (pp.d_b) cudaFree(pp.d_b);
        if (pp.d_bias) cudaFree(pp.d_bias);
        if (pp.d_table) cudaFree(pp.d_table);
        if (pp.d_scales) cudaFree(pp.d_scales);
        if (pp.h_scales) cudaFreeHost(pp.h_scales);
        if (h->d_status) cudaFree(h->d_status);
        if (h->d_prof) cudaFree(h->d_prof);
        (void)cudaGetLastError();
    }
    delete h;
    return SL8_OK;
}

SL8_API const char* sl8_last_error_string(sl8_handle_t h) {
    if (!h) return g_create_error.c_str();
    return h->err.c_str();
}

// =========================================================================== layers

SL8_API int sl8_patch_embed_fp8(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                                const float* scale_a, const float* scale_b, const void* table, int64_t ld_table,
                                int period, int table_rows, int row_phase, void* D, int64_t ldd, int64_t M, int N, int K,
                                unsigned flags, sl8_stream_t stream) {
    Problem q = {};
    q.op = SL8_OP_PATCH_EMBED; q.out_dtype = SL8_OUT_BF16;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb;
    q.scale_a = scale_a; q.scale_b = scale_b;
    q.side = table; q.ld_side = ld_table; q.period = period; q.row_phase = row_phase; q.table_rows = table_rows;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run(h, q, static_cast<cudaStream_t>(stream));
}

SL8_API int sl8_fc1_gelu_fp8(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                             const float* scale_a, const float* scale_b, const void* bias, void* D, int64_t ldd,
                             int out_dtype, const float* out_scale, int64_t M, int N, int K, unsigned flags,
                             sl8_stream_t stream) {
    Problem q = {};
    q.op = SL8_OP_FC1_GELU; q.out_dtype = out_dtype;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb;
    q.scale_a = scale_a; q.scale_b = scale_b; q.out_scale = out_scale;
    q.bias = bias;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run(h, q, static_cast<cudaStream_t>(stream));
}

SL8_API int sl8_linear_bias_fp8(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                                const float* scale_a, const float* scale_b, const void* bias, void* D, int64_t ldd,
                                int out_dtype, const float* out_scale, int64_t M, int N, int K, unsigned flags,
                                sl8_stream_t stream) {
    return sl8_fc1_gelu_fp8(h, A, lda, B, ldb, scale_a, scale_b, bias, D, ldd, out_dtype, out_scale, M, N, K,
                            flags | SL8_FLAG_NO_ACTIVATION, stream);
}

SL8_API int sl8_fc2_residual_fp8(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                                 const float* scale_a, const float* scale_b, const void* bias, const void* residual,
                                 int64_t ldr, void* D, int64_t ldd, int64_t M, int N, int K, unsigned flags,
                                 sl8_stream_t stream) {
    Problem q = {};
    q.op = SL8_OP_FC2_RESIDUAL; q.out_dtype = SL8_OUT_BF16;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb;
    q.scale_a = scale_a; q.scale_b = scale_b;
    q.bias = bias; q.side = residual; q.ld_side = ldr;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run(h, q, static_cast<cudaStream_t>(stream));
}

// =========================================================================== host operands

namespace {

int ensure(sl8_handle_t h, void** p, size_t* have, size_t need) {
    if (*have >= need && *p) return SL8_OK;
    if (*p) { cudaFree(*p); *p = nullptr; *have = 0; }
    cudaError_t e = cudaMalloc(p, need);
    if (e != cudaSuccess) return fail_cuda(h, e, "cudaMalloc(host-operand staging)");
    *have = need;
    return SL8_OK;
}

// Rows per slab: about 64 MiB of output, a multiple of 256 rows so slabs start on tile rows.
long long slab_rows_for(long long M, int N, int K, int out_bytes, bool has_res) {
    const double per_row = (double)K + (double)N * out_bytes + (has_res ? 2.0 * N : 0.0);
    long long rows = (long long)(64.0 * 1024 * 1024 / per_row);
    rows = (rows / 256) * 256;
    if (rows < 256) rows = 256;
    if (rows > M) rows = M;
    return rows;
}

int run_host(sl8_handle_t h, Problem q, float scale_a, float scale_b, float out_scale) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!q.A || !q.B || !q.D) return fail(h, SL8_ERR_INVALID_VALUE, "A, B and D must not be NULL");
    if (q.M < 1 || q.N < 1 || q.K < 1) return fail(h, SL8_ERR_INVALID_VALUE, "M, N, K must be positive");
    if (q.lda < q.K || q.ldb < q.K || q.ldd < q.N) return fail(h, SL8_ERR_INVALID_VALUE, "leading dimension too small");
    if (q.lda % 16 || q.ldb % 16) return fail(h, SL8_ERR_ALIGNMENT, "lda and ldb must be multiples of 16 bytes");
    const int ob = (q.out_dtype == SL8_OUT_BF16) ? 2 : 1;
    if ((q.ldd * ob) % 16) return fail(h, SL8_ERR_ALIGNMENT, "row pitch of D must be a multiple of 16 bytes");
    const bool has_res = q.op == SL8_OP_FC2_RESIDUAL;
    if (has_res && (!q.side || q.ld_side < q.N || (q.ld_side * 2) % 16)) return fail(h, SL8_ERR_INVALID_VALUE, "bad residual");
    if (q.op == SL8_OP_PATCH_EMBED && (!q.side || q.period < 1 || q.table_rows < q.period || q.ld_side < q.N || (q.ld_side * 2) % 16 || q.row_phase < 0))
        return fail(h, SL8_ERR_INVALID_VALUE, "bad table");

    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    HostPipe& pp = h->pipe;
    cudaError_t e;
    if (!pp.ready) {
        for (int i = 0; i < HostPipe::SLOTS; i++) {
            e = cudaStreamCreateWithFlags(&pp.stream[i], cudaStreamNonBlocking);
            if (e != cudaSuccess) return fail_cuda(h, e, "cudaStreamCreate");
        }
        e = cudaEventCreateWithFlags(&pp.consts_ready, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail_cuda(h, e, "cudaEventCreate");
        e = cudaMalloc(reinterpret_cast<void**>(&pp.d_scales), 16);
        if (e != cudaSuccess) return fail_cuda(h, e, "cudaMalloc(scales)");
        e = cudaMallocHost(reinterpret_cast<void**>(&pp.h_scales), 16);
        if (e != cudaSuccess) return fail_cuda(h, e, "cudaMallocHost(scales)");
        pp.ready = true;
    }
    const long long slab = slab_rows_for(q.M, q.N, q.K, ob, has_res);
    int rc;
    for (int i = 0; i < HostPipe::SLOTS; i++) {
        size_t ha = pp.a_bytes, hd = pp.d_bytes, hr = pp.r_bytes;
        if ((rc = ensure(h, &pp.d_a[i], &ha, (size_t)slab * q.lda)) != SL8_OK) return rc;
        if ((rc = ensure(h, &pp.d_d[i], &hd, (size_t)slab * q.ldd * ob)) != SL8_OK) return rc;
        if (has_res && (rc = ensure(h, &pp.d_r[i], &hr, (size_t)slab * q.ld_side * 2)) != SL8_OK) return rc;
        if (i == HostPipe::SLOTS - 1) { pp.a_bytes = ha; pp.d_bytes = hd; pp.r_bytes = hr; }
    }
    if ((rc = ensure(h, &pp.d_b, &pp.b_bytes, (size_t)q.N * q.ldb)) != SL8_OK) return rc;
    const size_t bias_need = (size_t)q.N * ((q.flags & SL8_FLAG_BIAS_F32) ? 4 : 2);
    if (q.bias && (rc = ensure(h, &pp.d_bias, &pp.bias_bytes, bias_need)) != SL8_OK) return rc;
    if (q.op == SL8_OP_PATCH_EMBED && (rc = ensure(h, &pp.d_table, &pp.table_bytes, (size_t)q.table_rows * q.ld_side * 2)) != SL8_OK) return rc;

    // constants, once per call, on slot 0's stream
    cudaStream_t s0 = pp.stream[0];
    pp.h_scales[0] = scale_a; pp.h_scales[1] = scale_b; pp.h_scales[2] = out_scale;
    cudaMemcpyAsync(pp.d_scales, pp.h_scales, 12, cudaMemcpyHostToDevice, s0);
    cudaMemcpyAsync(pp.d_b, q.B, (size_t)q.N * q.ldb, cudaMemcpyHostToDevice, s0);
    if (q.bias) cudaMemcpyAsync(pp.d_bias, q.bias, bias_need, cudaMemcpyHostToDevice, s0);
    if (q.op == SL8_OP_PATCH_EMBED) cudaMemcpyAsync(pp.d_table, q.side, (size_t)q.table_rows * q.ld_side * 2, cudaMemcpyHostToDevice, s0);
    e = cudaEventRecord(pp.consts_ready, s0);
    if (e != cudaSuccess) return fail_cuda(h, e, "upload of constants");

    const uint8_t* hA = static_cast<const uint8_t*>(q.A);
    const uint8_t* hR = static_cast<const uint8_t*>(q.side);
    uint8_t* hD = static_cast<uint8_t*>(q.D);
    int slot = 0;
    for (long long r0 = 0; r0 < q.M; r0 += slab, slot = (slot + 1) % HostPipe::SLOTS) {
        const long long rows = (r0 + slab < q.M) ? slab : q.M - r0;
        cudaStream_t s = pp.stream[slot];
        if (slot != 0 || r0 == 0) cudaStreamWaitEvent(s, pp.consts_ready, 0);
        cudaMemcpyAsync(pp.d_a[slot], hA + (size_t)r0 * q.lda, (size_t)rows * q.lda, cudaMemcpyHostToDevice, s);
        if (has_res) cudaMemcpyAsync(pp.d_r[slot], hR + (size_t)r0 * q.ld_side * 2, (size_t)rows * q.ld_side * 2, cudaMemcpyHostToDevice, s);
        Problem d = q;
        d.A = pp.d_a[slot];
        d.B = pp.d_b;
        d.D = pp.d_d[slot];
        d.M = rows;
        d.bias = q.bias ? pp.d_bias : nullptr;
        d.scale_a = pp.d_scales; d.scale_b = pp.d_scales + 1; d.out_scale = pp.d_scales + 2;
        if (q.op == SL8_OP_PATCH_EMBED) { d.side = pp.d_table; d.row_phase = (int)((q.row_phase + r0) % q.period); }
        if (has_res) d.side = pp.d_r[slot];
        rc = run(h, d, s);
        if (rc != SL8_OK) { cudaDeviceSynchronize(); return rc; }
        cudaMemcpyAsync(hD + (size_t)r0 * q.ldd * ob, pp.d_d[slot], (size_t)rows * q.ldd * ob, cudaMemcpyDeviceToHost, s);
    }
    for (int i = 0; i < HostPipe::SLOTS; i++) {
        e = cudaStreamSynchronize(pp.stream[i]);
        if (e != cudaSuccess) return fail_cuda(h, e, "host-operand pipeline");
    }
    return SL8_OK;
}

}  // namespace

SL8_API int sl8_patch_embed_fp8_host(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                                     float scale_a, float scale_b, const void* table, int64_t ld_table, int period,
                                     int table_rows, int row_phase, void* D, int64_t ldd, int64_t M, int N, int K,
                                     unsigned flags) {
    Problem q = {};
    q.op = SL8_OP_PATCH_EMBED; q.out_dtype = SL8_OUT_BF16;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb;
    q.side = table; q.ld_side = ld_table; q.period = period; q.row_phase = row_phase; q.table_rows = table_rows;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run_host(h, q, scale_a, scale_b, 1.0f);
}

SL8_API int sl8_fc1_gelu_fp8_host(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb, float scale_a,
                                  float scale_b, const void* bias, void* D, int64_t ldd, int out_dtype, float out_scale,
                                  int64_t M, int N, int K, unsigned flags) {
    if (out_dtype != SL8_OUT_BF16 && out_dtype != SL8_OUT_E4M3) return fail(h, SL8_ERR_INVALID_VALUE, "unknown out_dtype");
    Problem q = {};
    q.op = SL8_OP_FC1_GELU; q.out_dtype = out_dtype;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb; q.bias = bias;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run_host(h, q, scale_a, scale_b, out_scale);
}

SL8_API int sl8_fc2_residual_fp8_host(sl8_handle_t h, const void* A, int64_t lda, const void* B, int64_t ldb,
                                      float scale_a, float scale_b, const void* bias, const void* residual, int64_t ldr,
                                      void* D, int64_t ldd, int64_t M, int N, int K, unsigned flags) {
    Problem q = {};
    q.op = SL8_OP_FC2_RESIDUAL; q.out_dtype = SL8_OUT_BF16;
    q.A = A; q.B = B; q.lda = lda; q.ldb = ldb; q.bias = bias;
    q.side = residual; q.ld_side = ldr;
    q.D = D; q.ldd = ldd; q.M = M; q.N = N; q.K = K; q.flags = flags;
    return run_host(h, q, scale_a, scale_b, 1.0f);
}

// =========================================================================== dispatch

SL8_API int sl8_num_variants(void) { return SL8_NUM_VARIANTS; }

SL8_API int sl8_describe_variant(int variant_id, sl8_config* out) {
    const VariantEntry* v = variant(variant_id);
    if (!v || !out) return SL8_ERR_INVALID_VALUE;
    fill_config(v, sl8::K_FC1_BF16, 0, out);
    return SL8_OK;
}

SL8_API int sl8_query_config(sl8_handle_t h, int op, int out_dtype, int64_t M, int N, int K, sl8_config* out) {
    if (!out || M < 1 || N < 1 || K < 1 || op < 0 || op > 2) return SL8_ERR_INVALID_VALUE;
    int vid = (h && h->forced_variant >= 0) ? h->forced_variant : pick_variant(op, out_dtype, M, N, K);
    const VariantEntry* v = variant(vid);
    if (!v) return SL8_ERR_INVALID_VALUE;
    const int slot = kernel_slot(op, out_dtype);
    const int tile_m = 128 * v->cg;
    const long long nt = ((M + tile_m - 1) / tile_m) * ((N + v->tn - 1) / v->tn);
    const int sms = h ? h->sm_count : 148;
    long long clusters = sms / v->cg;
    if (nt < clusters) clusters = nt;
    fill_config(v, slot, (int)clusters * v->cg, out);
    return SL8_OK;
}

SL8_API int sl8_set_variant(sl8_handle_t h, int variant_id) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (variant_id >= SL8_NUM_VARIANTS) return fail(h, SL8_ERR_INVALID_VALUE, "no such kernel variant");
    std::lock_guard<std::mutex> lock(h->mu);
    h->forced_variant = variant_id < 0 ? -1 : variant_id;
    return SL8_OK;
}

// =========================================================================== watchdog

SL8_API int sl8_device_status(sl8_handle_t h, sl8_stream_t stream, unsigned detail[4]) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    DeviceGuard guard(h->device);
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail_cuda(h, e, "cudaStreamSynchronize");
    uint32_t st[4] = {0, 0, 0, 0};
    e = cudaMemcpy(st, h->d_status, 16, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(h, e, "read of the status block");
    if (detail) for (int i = 0; i < 4; i++) detail[i] = st[i];
    if (st[0] == 0) return SL8_OK;
    cudaMemset(h->d_status, 0, 16);
    char buf[160];
    static const char* names[] = {"", "producer waiting for a free stage", "MMA thread waiting for operands",
                                  "MMA thread waiting for a free accumulator", "epilogue waiting for an accumulator",
                                  "epilogue waiting for table / residual data"};
    snprintf(buf, sizeof buf, "device wait expired: %s (index %u, tile %u, block %u)", st[0] < 6 ? names[st[0]] : "?", st[1],
             st[2], st[3]);
    return fail(h, SL8_ERR_DEVICE_TIMEOUT, buf);
}

SL8_API int sl8_set_wait_budget_ms(sl8_handle_t h, int ms) {
    if (!h || ms < 1) return SL8_ERR_INVALID_VALUE;
    h->wait_budget_ms = static_cast<unsigned>(ms);
    return SL8_OK;
}

// =========================================================================== tracing

SL8_API int sl8_trace_enable(sl8_handle_t h, int on) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    if (on && !h->d_prof) {
        const int blocks = 2 * h->sm_count;
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&h->d_prof), sizeof(long long) * sl8::PROF_SLOTS * blocks);
        if (e != cudaSuccess) return fail_cuda(h, e, "cudaMalloc(tracing buffer)");
        cudaMemset(h->d_prof, 0, sizeof(long long) * sl8::PROF_SLOTS * blocks);
        h->prof_blocks = blocks;
    } else if (!on && h->d_prof) {
        cudaDeviceSynchronize();
        cudaFree(h->d_prof);
        h->d_prof = nullptr;
        h->prof_blocks = 0;
    }
    return SL8_OK;
}

SL8_API int sl8_trace_read(sl8_handle_t h, long long* out, int max_blocks) {
    if (!h || !out || max_blocks < 1) return SL8_ERR_INVALID_VALUE;
    if (!h->d_prof) return fail(h, SL8_ERR_INVALID_VALUE, "tracing is not enabled");
    DeviceGuard guard(h->device);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail_cuda(h, e, "cudaDeviceSynchronize");
    int n = h->last_grid < max_blocks ? h->last_grid : max_blocks;
    e = cudaMemcpy(out, h->d_prof, sizeof(long long) * sl8::PROF_SLOTS * n, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail_cuda(h, e, "read of the tracing buffer");
    return n;
}

// =========================================================================== periodic table

namespace {

__global__ void make_table_kernel(const float* __restrict__ bias, const float* __restrict__ pos, int period, int N,
                                  __nv_bfloat16* __restrict__ table, long long ld, int rows) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(rows) * N) return;
    const int r = static_cast<int>(idx / N), c = static_cast<int>(idx % N);
    const float b = bias ? bias[c] : 0.0f;
    table[r * ld + c] = __float2bfloat16(b + pos[static_cast<long long>(r % period) * N + c]);   // patch_embed.cu:96
}

__global__ void extend_table_kernel(const __nv_bfloat16* __restrict__ in, long long ld_in, int period, int N,
                                    __nv_bfloat16* __restrict__ out, long long ld_out, int rows) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(rows) * N) return;
    const int r = static_cast<int>(idx / N), c = static_cast<int>(idx % N);
    out[r * ld_out + c] = in[static_cast<long long>(r % period) * ld_in + c];
}

}  // namespace

SL8_API int sl8_padded_table_rows(int period) { return period < 1 ? 0 : (period + 127 + 31) / 32 * 32; }

SL8_API int sl8_make_periodic_table(sl8_handle_t h, const float* bias, const float* pos, int period, int N, void* table,
                                    int64_t ld_table, int rows_out, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!pos || !table || period < 1 || N < 1 || rows_out < 1 || ld_table < N) return fail(h, SL8_ERR_INVALID_VALUE, "bad table arguments");
    DeviceGuard guard(h->device);
    const long long total = static_cast<long long>(rows_out) * N;
    make_table_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        bias, pos, period, N, static_cast<__nv_bfloat16*>(table), ld_table, rows_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "table kernel launch");
}

SL8_API int sl8_extend_periodic_table(sl8_handle_t h, const void* table_in, int64_t ld_in, int period, int N,
                                      void* table_out, int64_t ld_out, int rows_out, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!table_in || !table_out || period < 1 || N < 1 || rows_out < 1 || ld_in < N || ld_out < N)
        return fail(h, SL8_ERR_INVALID_VALUE, "bad table arguments");
    DeviceGuard guard(h->device);
    const long long total = static_cast<long long>(rows_out) * N;
    extend_table_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(table_in), ld_in, period, N, static_cast<__nv_bfloat16*>(table_out), ld_out, rows_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "table kernel launch");
}

// =========================================================================== producer-side steps
// What feeds A: pixels -> patch rows (the Conv2d of the patch embedding written as a GEMM operand,
// docs/architecture.md:11-12 of the reference, which stops at the GEMM) with the per-tensor quantisation to
// e4m3 fused in, and the dynamic quantisation of a bf16 / fp32 activation (abs-max -> scale -> e4m3 codes)
// for a caller that has no static scale between FC1 and FC2.  Byte work bounded by HBM.

namespace {

__device__ __forceinline__ float prep_load(const float* p) { return __ldg(p); }
__device__ __forceinline__ float prep_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ uint8_t prep_e4m3(float v) { return static_cast<uint8_t>(sl8::pack_e4m3x2(v, 0.0f) & 0xFFu); }

// One block per (image, patch row): the C * P image rows of that strip are read with coalesced loads, quantised,
// placed in shared memory at the position they have in the strip's `gw` rows of A (column c * P * P + py * P + px,
// the flattening order of a Conv2d weight [N, C, P, P]) and those rows are then written whole, pad included.
template <typename PT>
__global__ void patchify_quantize_kernel(const PT* __restrict__ pixels, int C, int H, int W, int P, int gh, int gw,
                                         const float* __restrict__ scale, uint8_t* __restrict__ A, long long lda,
                                         int row_bytes) {
    extern __shared__ __align__(16) uint8_t prep_tile[];
    const int img = blockIdx.x / gh, gy = blockIdx.x - img * gh;
    const int K = C * P * P;
    const float inv = __frcp_rn(scale ? __ldg(scale) : 1.0f);
    for (int i = threadIdx.x; i < gw * (row_bytes - K); i += blockDim.x)          // the zero pad K .. row_bytes
        prep_tile[(i / (row_bytes - K)) * row_bytes + K + i % (row_bytes - K)] = 0;
    // A warp per image row (c, gy * P + py) of the strip; its lanes read the row with consecutive 8-byte loads (two
    // pixels each) and drop the two codes into the patch row they belong to.  Odd P or W: one pixel at a time.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int strip = gw * P;
    const bool pairs = (P % 2 == 0) && (W % 2 == 0);
    for (int cp = warp; cp < C * P; cp += nwarps) {
        const int py = cp % P, c = cp / P;
        const PT* src = pixels + ((static_cast<long long>(img) * C + c) * H + (gy * P + py)) * W;
        uint8_t* dst = prep_tile + c * P * P + py * P;
        if (pairs) {
            for (int x = 2 * lane; x < strip; x += 64) {
                float a, b;
                if constexpr (sizeof(PT) == 4) {
                    const float2 v = __ldg(reinterpret_cast<const float2*>(src + x));
                    a = v.x; b = v.y;
                } else {
                    const uint32_t w = __ldg(reinterpret_cast<const unsigned*>(src + x));
                    a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xFFFF0000u);
                }
                const int gx = x / P, px = x - gx * P;
                *reinterpret_cast<uint16_t*>(dst + gx * row_bytes + px) = sl8::pack_e4m3x2(a * inv, b * inv);
            }
        } else {
            for (int x = lane; x < strip; x += 32) {
                const int gx = x / P, px = x - gx * P;
                dst[gx * row_bytes + px] = prep_e4m3(prep_load(src + x) * inv);
            }
        }
    }
    __syncthreads();
    const long long m0 = (static_cast<long long>(img) * gh + gy) * gw;
    const int vecs = row_bytes / 16;
    for (int i = threadIdx.x; i < gw * vecs; i += blockDim.x) {
        const int r = i / vecs, v = i - r * vecs;
        *reinterpret_cast<uint4*>(A + (m0 + r) * lda + 16 * v) = *reinterpret_cast<const uint4*>(prep_tile + r * row_bytes + 16 * v);
    }
}

// |x| of non-negative floats orders like their bit patterns: one atomicMax on the bits per block.
template <typename T>
__device__ __forceinline__ float prep_absmax8(const T* p) {          // max |.| of eight consecutive elements, 16-byte loads
    float m;
    if constexpr (sizeof(T) == 4) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
        m = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                  fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
    } else {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        m = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++)
            m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xFFFF0000u))));
    }
    return m;
}

// `vectors` != 0: rows of cols = 8 * vectors_per_row elements on 16-byte boundaries, eight elements per load;
// otherwise element by element.
template <typename T>
__global__ void amax_kernel(const T* __restrict__ x, long long rows, int cols, long long ld, int vectors,
                            unsigned* __restrict__ amax_bits) {
    float m = 0.0f;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vectors) {
        const int vpr = cols / 8;
        const long long total = rows * vpr;
        if (ld == cols) {
            for (long long i = first; i < total; i += stride) m = fmaxf(m, prep_absmax8(x + 8 * i));
        } else {
            for (long long i = first; i < total; i += stride) {
                const long long r = i / vpr;
                m = fmaxf(m, prep_absmax8(x + r * ld + 8 * (i - r * vpr)));
            }
        }
    } else {
        const long long total = rows * cols;
        for (long long i = first; i < total; i += stride) {
            const long long r = i / cols;
            m = fmaxf(m, fabsf(prep_load(x + r * ld + (i - r * cols))));
        }
    }
    unsigned b = __reduce_max_sync(0xffffffffu, __float_as_uint(m));
    __shared__ unsigned warp_max[32];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x < 32) {
        b = threadIdx.x < (blockDim.x + 31) / 32 ? warp_max[threadIdx.x] : 0u;
        b = __reduce_max_sync(0xffffffffu, b);
        if (threadIdx.x == 0) atomicMax(amax_bits, b);
    }
}

__global__ void scale_from_amax_kernel(const unsigned* __restrict__ amax_bits, float* __restrict__ scale) {
    const float a = __uint_as_float(*amax_bits);
    *scale = a > 0.0f ? a / 448.0f : 1.0f;                 // 448 = largest e4m3 value; an all-zero tensor keeps scale 1
}

template <typename T>
__device__ __forceinline__ void ln_load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void ln_load8<float>(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void ln_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}

template <typename T>
__global__ void quantize_e4m3_kernel(const T* __restrict__ x, long long rows, int cols, long long ld,
                                     const float* __restrict__ scale, uint8_t* __restrict__ out, long long ld_out) {
    const float inv = __frcp_rn(scale ? __ldg(scale) : 1.0f);
    const int groups = (cols + 7) / 8;                      // eight columns per thread: one 8-byte store
    const long long total = rows * groups;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / groups;
        const int c0 = static_cast<int>(i - r * groups) * 8;
        const T* src = x + r * ld + c0;
        uint8_t* dst = out + r * ld_out + c0;
        if (c0 + 8 <= cols && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
            float v[8];
            ln_load8<T>(src, v);
            uint32_t w[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; h2++)
                w[h2] = static_cast<uint32_t>(sl8::pack_e4m3x2(v[4 * h2] * inv, v[4 * h2 + 1] * inv)) |
                        (static_cast<uint32_t>(sl8::pack_e4m3x2(v[4 * h2 + 2] * inv, v[4 * h2 + 3] * inv)) << 16);
            *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
        } else {
            for (int c = c0; c < cols && c < c0 + 8; c++) dst[c - c0] = prep_e4m3(prep_load(src + (c - c0)) * inv);
        }
    }
}

int prep_grid(sl8_handle_t h, long long work_items) {
    const long long want = (work_items + 255) / 256;
    const long long cap = static_cast<long long>(h->sm_count > 0 ? h->sm_count : 148) * 16;   // a multiple of the SM count
    return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace

SL8_API int sl8_patchify_quantize_e4m3(sl8_handle_t h, const void* pixels, int pixel_dtype, int images, int channels,
                                       int height, int width, int patch, const float* scale, void* A, int64_t lda,
                                       sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!pixels || !A || images < 1 || channels < 1 || patch < 1 || height < patch || width < patch)
        return fail(h, SL8_ERR_INVALID_VALUE, "bad patchify arguments");
    if (pixel_dtype != SL8_DT_F32 && pixel_dtype != SL8_DT_BF16) return fail(h, SL8_ERR_INVALID_VALUE, "unknown pixel dtype");
    const int K = channels * patch * patch, gh = height / patch, gw = width / patch;
    if (lda < K) return fail(h, SL8_ERR_INVALID_VALUE, "lda smaller than channels * patch * patch");
    if (!aligned16(A) || lda % 16 != 0) return fail(h, SL8_ERR_ALIGNMENT, "A and lda must be multiples of 16 bytes");
    if (!aligned16(pixels)) return fail(h, SL8_ERR_ALIGNMENT, "pixels must be 16-byte aligned");
    // whole rows are written when the pad is short (K = 588 at pitch 640), else K rounded up to 16 bytes
    const int row_bytes = static_cast<int>(lda - K < 128 ? lda : (K + 15) / 16 * 16);
    const size_t smem = static_cast<size_t>(gw) * row_bytes;
    if (smem > 200 * 1024) return fail(h, SL8_ERR_UNSUPPORTED, "one strip of patches exceeds 200 KiB of shared memory");
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaSuccess;
    const unsigned grid = static_cast<unsigned>(images) * gh;
    if (pixel_dtype == SL8_DT_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(patchify_quantize_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            patchify_quantize_kernel<float><<<grid, 256, smem, s>>>(static_cast<const float*>(pixels), channels, height, width, patch,
                                                                    gh, gw, scale, static_cast<uint8_t*>(A), lda, row_bytes);
    } else {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(patchify_quantize_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            patchify_quantize_kernel<__nv_bfloat16><<<grid, 256, smem, s>>>(static_cast<const __nv_bfloat16*>(pixels), channels, height,
                                                                            width, patch, gh, gw, scale, static_cast<uint8_t*>(A), lda, row_bytes);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "patchify kernel launch");
}

SL8_API int sl8_amax_scale(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld, float* amax,
                           float* scale, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!x || !amax || rows < 1 || cols < 1 || ld < cols) return fail(h, SL8_ERR_INVALID_VALUE, "bad amax arguments");
    if (dtype != SL8_DT_F32 && dtype != SL8_DT_BF16) return fail(h, SL8_ERR_INVALID_VALUE, "unknown dtype");
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(amax, 0, sizeof(float), s);
    if (e != cudaSuccess) return fail_cuda(h, e, "cudaMemsetAsync(amax)");
    const int grid = prep_grid(h, rows * cols / 8);
    const int vectors = (cols % 8 == 0 && ld % 8 == 0 && aligned16(x)) ? 1 : 0;
    if (dtype == SL8_DT_F32)
        amax_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), rows, cols, ld, vectors, reinterpret_cast<unsigned*>(amax));
    else
        amax_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, vectors,
                                                        reinterpret_cast<unsigned*>(amax));
    if (scale) scale_from_amax_kernel<<<1, 1, 0, s>>>(reinterpret_cast<const unsigned*>(amax), scale);
    e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "amax kernel launch");
}

SL8_API int sl8_quantize_e4m3(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld, const float* scale,
                              void* out, int64_t ld_out, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!x || !out || rows < 1 || cols < 1 || ld < cols || ld_out < cols) return fail(h, SL8_ERR_INVALID_VALUE, "bad quantize arguments");
    if (dtype != SL8_DT_F32 && dtype != SL8_DT_BF16) return fail(h, SL8_ERR_INVALID_VALUE, "unknown dtype");
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = prep_grid(h, rows * ((cols + 7) / 8));
    if (dtype == SL8_DT_F32)
        quantize_e4m3_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), rows, cols, ld, scale, static_cast<uint8_t*>(out), ld_out);
    else
        quantize_e4m3_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, scale,
                                                                 static_cast<uint8_t*>(out), ld_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "quantize kernel launch");
}

// ---- LayerNorm -> quantise: the prologue of FC1 (docs/architecture.md:92-101 of the reference lists it as unstarted).
// One warp per row: mean, variance (two passes, fp32, the row stays in L1 after the first), then
// e4m3((x - mean) * rsqrt(var + eps) * gamma + beta) * (1 / scale), eight columns per lane and step.
namespace {

// CHUNKS > 0: cols <= 256 * CHUNKS and the lane keeps its 8 * CHUNKS elements in registers (x is read once);
// CHUNKS == 0: any width, three passes over the row (the second and third hit L1 / L2).  Scalar fp32 arithmetic:
// the packed two-element forms were measured 20 - 40 % slower here.
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(256, 3) layernorm_quantize_kernel(const T* __restrict__ x, long long rows, int cols, long long ld,
                                          const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                                          const float* __restrict__ scale, uint8_t* __restrict__ out, long long ld_out) {
    const int lane = threadIdx.x & 31;
    const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    const float inv = __frcp_rn(scale ? __ldg(scale) : 1.0f);
    const float inv_n = 1.0f / static_cast<float>(cols);
    constexpr int NC = CHUNKS > 0 ? CHUNKS : 1;
    for (long long r = warp; r < rows; r += warps) {
        const T* row = x + r * ld;
        float v[NC][8];
        float sum = 0.0f;
        if constexpr (CHUNKS > 0) {
#pragma unroll
            for (int j = 0; j < NC; j++) {
                const int c = lane * 8 + 256 * j;
                if (c < cols) {
                    ln_load8<T>(row + c, v[j]);
#pragma unroll
                    for (int i = 0; i < 8; i++) sum += v[j][i];
                }
            }
        } else {
            for (int c = lane * 8; c < cols; c += 256) {
                ln_load8<T>(row + c, v[0]);
#pragma unroll
                for (int i = 0; i < 8; i++) sum += v[0][i];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_n;
        float sq = 0.0f;
        if constexpr (CHUNKS > 0) {
#pragma unroll
            for (int j = 0; j < NC; j++)
                if (lane * 8 + 256 * j < cols) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        v[j][i] -= mean;                                   // x - mean, kept for the output pass
                        sq = fmaf(v[j][i], v[j][i], sq);
                    }
                }
        } else {
            for (int c = lane * 8; c < cols; c += 256) {
                ln_load8<T>(row + c, v[0]);
#pragma unroll
                for (int i = 0; i < 8; i++) sq = fmaf(v[0][i] - mean, v[0][i] - mean, sq);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = rsqrtf(sq * inv_n + eps);
        // d = x - mean -> ((d * rstd) * gamma + beta) * (1 / scale) -> eight e4m3 codes, one 8-byte store
        auto emit = [&](const float (&d)[8], int c) {
            float g[8], b[8], y[8];
            if (gamma) ln_load8<float>(gamma + c, g);
            if (beta) ln_load8<float>(beta + c, b);
#pragma unroll
            for (int i = 0; i < 8; i++) y[i] = fmaf(d[i] * rstd, gamma ? g[i] : 1.0f, beta ? b[i] : 0.0f) * inv;
            const uint32_t lo = static_cast<uint32_t>(sl8::pack_e4m3x2(y[0], y[1])) | (static_cast<uint32_t>(sl8::pack_e4m3x2(y[2], y[3])) << 16);
            const uint32_t hi = static_cast<uint32_t>(sl8::pack_e4m3x2(y[4], y[5])) | (static_cast<uint32_t>(sl8::pack_e4m3x2(y[6], y[7])) << 16);
            *reinterpret_cast<uint2*>(out + r * ld_out + c) = make_uint2(lo, hi);
        };
        if constexpr (CHUNKS > 0) {
#pragma unroll
            for (int j = 0; j < NC; j++)
                if (lane * 8 + 256 * j < cols) emit(v[j], lane * 8 + 256 * j);
        } else {
            for (int c = lane * 8; c < cols; c += 256) {
                ln_load8<T>(row + c, v[0]);
#pragma unroll
                for (int i = 0; i < 8; i++) v[0][i] -= mean;
                emit(v[0], c);
            }
        }
    }
}

template <typename T>
void launch_layernorm(int grid, cudaStream_t s, const T* x, long long rows, int cols, long long ld, const float* gamma,
                      const float* beta, float eps, const float* scale, uint8_t* out, long long ld_out) {
    if (cols <= 1280) layernorm_quantize_kernel<T, 5><<<grid, 256, 0, s>>>(x, rows, cols, ld, gamma, beta, eps, scale, out, ld_out);
    else if (cols <= 2048) layernorm_quantize_kernel<T, 8><<<grid, 256, 0, s>>>(x, rows, cols, ld, gamma, beta, eps, scale, out, ld_out);
    else layernorm_quantize_kernel<T, 0><<<grid, 256, 0, s>>>(x, rows, cols, ld, gamma, beta, eps, scale, out, ld_out);
}

}  // namespace

SL8_API int sl8_layernorm_quantize_e4m3(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld,
                                        const float* gamma, const float* beta, float eps, const float* scale, void* out,
                                        int64_t ld_out, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!x || !out || rows < 1 || cols < 1 || ld < cols || ld_out < cols || !(eps >= 0.0f))
        return fail(h, SL8_ERR_INVALID_VALUE, "bad layernorm arguments");
    if (dtype != SL8_DT_F32 && dtype != SL8_DT_BF16) return fail(h, SL8_ERR_INVALID_VALUE, "unknown dtype");
    if (cols % 8 != 0 || ld % 8 != 0 || ld_out % 8 != 0) return fail(h, SL8_ERR_UNSUPPORTED, "cols, ld and ld_out must be multiples of 8");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(out) & 7u) != 0 || (gamma && !aligned16(gamma)) || (beta && !aligned16(beta)))
        return fail(h, SL8_ERR_ALIGNMENT, "x, gamma, beta must be 16-byte aligned and out 8-byte aligned");
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int grid = prep_grid(h, rows * 32);            // one warp per row, eight warps per block
    if (dtype == SL8_DT_F32)
        launch_layernorm<float>(grid, s, static_cast<const float*>(x), rows, cols, ld, gamma, beta, eps, scale, static_cast<uint8_t*>(out), ld_out);
    else
        launch_layernorm<__nv_bfloat16>(grid, s, static_cast<const __nv_bfloat16*>(x), rows, cols, ld, gamma, beta, eps, scale,
                                        static_cast<uint8_t*>(out), ld_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? SL8_OK : fail_cuda(h, e, "layernorm kernel launch");
}
