// sl8_api.cu -- the C ABI of libsiglip_fp8.so (include/siglip_fp8.h): handle life cycle,
// argument validation, tensor-map encoding, the dispatch table and the launches.
//
// This file plays the part of the host half of each reference layer's main()
// (patch_embed.cu:104-246, fc1_gelu.cu:52-170, fc2.cu:72-200): it builds the three tensor
// maps, raises the dynamic shared-memory limit and launches the persistent kernel -- for
// run-time shapes, and returning status codes instead of exiting.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "sl8_internal.h"
#include "sl8_dispatch_table.h"

namespace {

using sl8::KernelParams;
using sl8::VariantEntry;
typedef sl8_encode_tiled_fn encode_tiled_fn;
typedef Sl8HostPipe HostPipe;
typedef Sl8MapCacheEntry MapCacheEntry;
typedef Sl8DeviceGuard DeviceGuard;

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

}  // namespace

int sl8_fail(sl8_handle_t h, int code, const std::string& msg) {
    if (h) h->err = msg;
    else g_create_error = msg;
    return code;
}

int sl8_fail_cuda(sl8_handle_t h, cudaError_t e, const char* what) {
    return sl8_fail(h, SL8_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

namespace {

inline int fail(sl8_handle_t h, int code, const std::string& msg) { return sl8_fail(h, code, msg); }
inline int fail_cuda(sl8_handle_t h, cudaError_t e, const char* what) { return sl8_fail_cuda(h, e, what); }
inline bool aligned16(const void* p) { return sl8_aligned16(p); }

// ---- dispatch -------------------------------------------------------------------------
// The table is generated from a sweep on B200 (python -m siglip_b200.sweep); shapes it does not hold fall back
// to rules (one line per rule; the first match wins).
int kernel_slot(int op, int out_dtype) {
    if (op == SL8_OP_PATCH_EMBED) return sl8::K_PE;
    if (op == SL8_OP_FC2_RESIDUAL) return sl8::K_FC2;
    return out_dtype == SL8_OUT_E4M3 ? sl8::K_FC1_E4M3 : sl8::K_FC1_BF16;
}

int pick_variant_exact_gelu(int op, int out_dtype, long long M, int N, int K);

// The sweep and the rules below are for the full epilogues.  An FC1 call whose epilogue is light (no activation: the
// Q / K / V projections; or the one-SFU-operation GELU) does not need sixteen epilogue warps to hide the SFU chain and
// runs faster on eight with the same ring depth (So400m FC1 shape, 46 656 rows: 198 against 220 us without activation,
// 207 against 221 us with the hardware tanh).
int pick_variant(int op, int out_dtype, long long M, int N, int K, unsigned flags) {
    const int v = pick_variant_exact_gelu(op, out_dtype, M, N, K);
    if (op == SL8_OP_FC1_GELU && (flags & (SL8_FLAG_NO_ACTIVATION | SL8_FLAG_GELU_HW_TANH)) && variant(v) && variant(v)->epi_warps == 16)
        return 2;
    return v;
}

int pick_variant_exact_gelu(int op, int out_dtype, long long M, int N, int K) {
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
    if (op == SL8_OP_FC1_GELU) return 15;     // GELU epilogue: four epilogue warps per scheduler
    if (op == SL8_OP_PATCH_EMBED) return 17;  // short K: eight epilogue warps, three staging boxes per column group, four stages
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
              unsigned box_outer, CUtensorMapL2promotion promo, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    for (int i = 0; i < sl8_context::kMapCache; i++) {      // callers hold h->mu
        const MapCacheEntry& c = h->map_cache[i];
        if (c.base == base && c.dt == (int)dt && c.promo == (int)promo && c.inner == inner && c.outer == outer &&
            c.pitch == pitch_bytes && c.box_inner == box_inner && c.box_outer == box_outer && c.swizzle == (int)swizzle) {
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
                           swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        MapCacheEntry& c = h->map_cache[h->map_cache_next];
        h->map_cache_next = (h->map_cache_next + 1) % sl8_context::kMapCache;
        c.dt = (int)dt; c.promo = (int)promo; c.base = base; c.inner = inner; c.outer = outer; c.pitch = pitch_bytes;
        c.box_inner = box_inner; c.box_outer = box_outer; c.swizzle = (int)swizzle; c.map = *map;
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

    int vid = h->forced_variant >= 0 ? h->forced_variant : pick_variant(q.op, q.out_dtype, q.M, q.N, q.K, q.flags);
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

    CUtensorMap map_a, map_b, map_bt, map_d;
    rc = encode_2d(h, &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.A, (unsigned long long)q.K, (unsigned long long)q.M,
                   (unsigned long long)q.lda, 128, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (rc != SL8_OK) return rc;
    rc = encode_2d(h, &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.B, (unsigned long long)q.K, (unsigned long long)q.N,
                   (unsigned long long)q.ldb, 128, (unsigned)(v->tn / v->cg), CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != SL8_OK) return rc;
    // The last N tile is as wide as what is left of N (a multiple of 16): its MMAs run with that N and each CTA
    // brings tail / cta_group rows of B per k-block through a second map with a box of that height.
    const int tail_cols = q.N % v->tn == 0 ? v->tn : q.N % v->tn;
    map_bt = map_b;
    if (tail_cols != v->tn) {
        rc = encode_2d(h, &map_bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q.B, (unsigned long long)q.K, (unsigned long long)q.N,
                       (unsigned long long)q.ldb, 128, (unsigned)(tail_cols / v->cg), CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (rc != SL8_OK) return rc;
    }
    // Staging rows (= store boxes) are 128 bytes wide, 64 where one epilogue warp's columns fill no more.
    const int row_bytes = (v->tn / (v->epi_warps / 4)) * ob < 128 ? 64 : 128;
    rc = encode_2d(h, &map_d, ob == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, ob, q.D,
                   (unsigned long long)q.N, (unsigned long long)q.M, (unsigned long long)q.ldd * ob,
                   (unsigned)(row_bytes / ob), 32, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
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
    p.tail_cols = tail_cols;
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
    p.flags = q.flags | (h->trace_coarse ? sl8::FLAG_COARSE_TRACE : 0u) | (h->single_acc ? sl8::FLAG_SINGLE_ACC : 0u) |
              (h->test_drop_b ? sl8::FLAG_TEST_DROP_B : 0u);
    p.wait_budget_us = h->wait_budget_us;
    p.status = h->d_status;
    p.prof = h->d_prof;

    const int grid = grid_for(h, v, slot, p.num_tiles);
    h->last_grid = grid;
    if (h->d_prof && grid > h->prof_blocks) return fail(h, SL8_ERR_INVALID_VALUE, "tracing buffer smaller than the grid");
    cudaError_t e = v->launch[slot](&map_a, &map_b, &map_bt, &map_d, &map_s, &p, grid, stream);
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
    const char* td = getenv("SL8_TEST_DROP_B");      // test aid: see FLAG_TEST_DROP_B
    h->test_drop_b = td && *td == '1';
    const char* sa = getenv("SL8_SINGLE_ACC");
    h->single_acc = sa && *sa == '1';
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
            if (pp.d_h[i]) cudaFree(pp.d_h[i]);
            if (pp.stream[i]) cudaStreamDestroy(pp.stream[i]);
        }
        if (pp.consts_ready) cudaEventDestroy(pp.consts_ready);
        if (pp.d_b) cudaFree(pp.d_b);
        if (pp.d_bias) cudaFree(pp.d_bias);
        if (pp.d_b2) cudaFree(pp.d_b2);
        if (pp.d_bias2) cudaFree(pp.d_bias2);
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

// Streams, the constants-uploaded event and the scale staging of the host-operand pipeline, created on first use.
int pipe_init(sl8_handle_t h) {
    HostPipe& pp = h->pipe;
    if (pp.ready) return SL8_OK;
    cudaError_t e;
    for (int i = 0; i < HostPipe::SLOTS; i++) {
        if (!pp.stream[i] && (e = cudaStreamCreateWithFlags(&pp.stream[i], cudaStreamNonBlocking)) != cudaSuccess) return fail_cuda(h, e, "cudaStreamCreate");
    }
    if (!pp.consts_ready && (e = cudaEventCreateWithFlags(&pp.consts_ready, cudaEventDisableTiming)) != cudaSuccess) return fail_cuda(h, e, "cudaEventCreate");
    if (!pp.d_scales && (e = cudaMalloc(reinterpret_cast<void**>(&pp.d_scales), 16)) != cudaSuccess) return fail_cuda(h, e, "cudaMalloc(scales)");
    if (!pp.h_scales && (e = cudaMallocHost(reinterpret_cast<void**>(&pp.h_scales), 16)) != cudaSuccess) return fail_cuda(h, e, "cudaMallocHost(scales)");
    pp.ready = true;
    return SL8_OK;
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

    // One host call at a time per handle: the staging buffers and the three streams belong to the call that runs.
    // (run() takes h->mu for the launch itself, so this is a second, outer lock.)
    std::lock_guard<std::mutex> pipe_lock(h->pipe_mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    HostPipe& pp = h->pipe;
    cudaError_t e;
    int rc = pipe_init(h);
    if (rc != SL8_OK) return rc;
    const long long slab = slab_rows_for(q.M, q.N, q.K, ob, has_res);
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

    // A copy or wait that cannot be enqueued ends the call: what was enqueued before it is drained first, so no
    // copy is still writing into the caller's buffers when the error is returned.
    auto bail = [&](cudaError_t err, const char* what) {
        cudaDeviceSynchronize();
        (void)cudaGetLastError();
        return fail_cuda(h, err, what);
    };
    // constants, once per call, on slot 0's stream
    cudaStream_t s0 = pp.stream[0];
    pp.h_scales[0] = scale_a; pp.h_scales[1] = scale_b; pp.h_scales[2] = out_scale;
    if ((e = cudaMemcpyAsync(pp.d_scales, pp.h_scales, 12, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of the scales");
    if ((e = cudaMemcpyAsync(pp.d_b, q.B, (size_t)q.N * q.ldb, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of B");
    if (q.bias && (e = cudaMemcpyAsync(pp.d_bias, q.bias, bias_need, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of the bias");
    if (q.op == SL8_OP_PATCH_EMBED &&
        (e = cudaMemcpyAsync(pp.d_table, q.side, (size_t)q.table_rows * q.ld_side * 2, cudaMemcpyHostToDevice, s0)) != cudaSuccess)
        return bail(e, "upload of the table");
    if ((e = cudaEventRecord(pp.consts_ready, s0)) != cudaSuccess) return bail(e, "upload of constants");

    const uint8_t* hA = static_cast<const uint8_t*>(q.A);
    const uint8_t* hR = static_cast<const uint8_t*>(q.side);
    uint8_t* hD = static_cast<uint8_t*>(q.D);
    int slot = 0;
    for (long long r0 = 0; r0 < q.M; r0 += slab, slot = (slot + 1) % HostPipe::SLOTS) {
        const long long rows = (r0 + slab < q.M) ? slab : q.M - r0;
        cudaStream_t s = pp.stream[slot];
        if ((slot != 0 || r0 == 0) && (e = cudaStreamWaitEvent(s, pp.consts_ready, 0)) != cudaSuccess) return bail(e, "wait for the constants");
        if ((e = cudaMemcpyAsync(pp.d_a[slot], hA + (size_t)r0 * q.lda, (size_t)rows * q.lda, cudaMemcpyHostToDevice, s)) != cudaSuccess)
            return bail(e, "upload of a slab of A");
        if (has_res && (e = cudaMemcpyAsync(pp.d_r[slot], hR + (size_t)r0 * q.ld_side * 2, (size_t)rows * q.ld_side * 2, cudaMemcpyHostToDevice, s)) != cudaSuccess)
            return bail(e, "upload of a slab of the residual");
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
        if ((e = cudaMemcpyAsync(hD + (size_t)r0 * q.ldd * ob, pp.d_d[slot], (size_t)rows * q.ldd * ob, cudaMemcpyDeviceToHost, s)) != cudaSuccess)
            return bail(e, "download of a slab of D");
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

// =========================================================================== FC1 -> FC2 chain

namespace {

struct ChainArgs {
    const void* A; long long lda;
    const void* W1; long long ldw1; const void* bias1;
    const void* W2; long long ldw2; const void* bias2;
    const void* residual; long long ldr;
    void* D; long long ldd;
    long long M; int d_model, d_ff;
    unsigned flags;
};

// The two launches of the MLP on device operands: hidden = e4m3(gelu(A.W1^T + b1) / hidden_scale), D = hidden.W2^T + b2 + R.
int run_chain(sl8_handle_t h, const ChainArgs& c, const float* scale_a, const float* scale_w1, const float* scale_w2,
              const float* hidden_scale, void* hidden, long long ld_hidden, cudaStream_t stream) {
    if (!hidden || !hidden_scale) return fail(h, SL8_ERR_INVALID_VALUE, "hidden buffer and hidden_scale must not be NULL");
    if (c.flags & ~(unsigned)(SL8_FLAG_BIAS_F32 | SL8_FLAG_GELU_HW_TANH)) return fail(h, SL8_ERR_INVALID_VALUE, "unknown flag bits");
    Problem q1 = {};
    q1.op = SL8_OP_FC1_GELU; q1.out_dtype = SL8_OUT_E4M3;
    q1.A = c.A; q1.lda = c.lda; q1.B = c.W1; q1.ldb = c.ldw1;
    q1.scale_a = scale_a; q1.scale_b = scale_w1; q1.out_scale = hidden_scale;
    q1.bias = c.bias1;
    q1.D = hidden; q1.ldd = ld_hidden; q1.M = c.M; q1.N = c.d_ff; q1.K = c.d_model; q1.flags = c.flags;
    int rc = run(h, q1, stream);
    if (rc != SL8_OK) return rc;
    Problem q2 = {};
    q2.op = SL8_OP_FC2_RESIDUAL; q2.out_dtype = SL8_OUT_BF16;
    q2.A = hidden; q2.lda = ld_hidden; q2.B = c.W2; q2.ldb = c.ldw2;
    q2.scale_a = hidden_scale; q2.scale_b = scale_w2;
    q2.bias = c.bias2; q2.side = c.residual; q2.ld_side = c.ldr;
    q2.D = c.D; q2.ldd = c.ldd; q2.M = c.M; q2.N = c.d_model; q2.K = c.d_ff; q2.flags = c.flags & SL8_FLAG_BIAS_F32;
    return run(h, q2, stream);
}

}  // namespace

SL8_API int sl8_mlp_chain_fp8(sl8_handle_t h, const void* A, int64_t lda, const void* W1, int64_t ldw1,
                              const float* scale_a, const float* scale_w1, const void* bias1, void* hidden,
                              int64_t ld_hidden, const float* hidden_scale, const void* W2, int64_t ldw2,
                              const float* scale_w2, const void* bias2, const void* residual, int64_t ldr, void* D,
                              int64_t ldd, int64_t M, int d_model, int d_ff, unsigned flags, sl8_stream_t stream) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    ChainArgs c = {A, lda, W1, ldw1, bias1, W2, ldw2, bias2, residual, ldr, D, ldd, M, d_model, d_ff, flags};
    return run_chain(h, c, scale_a, scale_w1, scale_w2, hidden_scale, hidden, ld_hidden, static_cast<cudaStream_t>(stream));
}

SL8_API int sl8_mlp_chain_fp8_host(sl8_handle_t h, const void* A, int64_t lda, const void* W1, int64_t ldw1, float scale_a,
                                   float scale_w1, const void* bias1, float hidden_scale, const void* W2, int64_t ldw2,
                                   float scale_w2, const void* bias2, const void* residual, int64_t ldr, void* D,
                                   int64_t ldd, int64_t M, int d_model, int d_ff, unsigned flags) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    if (!A || !W1 || !W2 || !residual || !D) return fail(h, SL8_ERR_INVALID_VALUE, "A, W1, W2, residual and D must not be NULL");
    if (M < 1 || d_model < 1 || d_ff < 1) return fail(h, SL8_ERR_INVALID_VALUE, "M, d_model, d_ff must be positive");
    if (lda < d_model || ldw1 < d_model || ldw2 < d_ff || ldr < d_model || ldd < d_model) return fail(h, SL8_ERR_INVALID_VALUE, "leading dimension too small");
    if (lda % 16 || ldw1 % 16 || ldw2 % 16 || (ldr * 2) % 16 || (ldd * 2) % 16) return fail(h, SL8_ERR_ALIGNMENT, "row pitches must be multiples of 16 bytes");
    if (!(hidden_scale > 0.0f)) return fail(h, SL8_ERR_INVALID_VALUE, "hidden_scale must be positive");

    std::lock_guard<std::mutex> pipe_lock(h->pipe_mu);
    DeviceGuard guard(h->device);
    if (!guard.ok) return fail(h, SL8_ERR_CUDA, "cudaSetDevice failed");
    HostPipe& pp = h->pipe;
    int rc = pipe_init(h);
    if (rc != SL8_OK) return rc;
    // Rows per slab: about 64 MiB of traffic over the bus (A up, residual up, D down); the hidden slab stays on the GPU.
    const long long ld_hidden = ((long long)d_ff + 127) / 128 * 128;
    long long slab = (long long)(64.0 * 1024 * 1024 / ((double)d_model * 5.0));
    slab = slab / 256 * 256;
    if (slab < 256) slab = 256;
    if (slab > M) slab = M;
    for (int i = 0; i < HostPipe::SLOTS; i++) {
        size_t ha = pp.a_bytes, hd = pp.d_bytes, hr = pp.r_bytes, hh = pp.h_bytes;
        if ((rc = ensure(h, &pp.d_a[i], &ha, (size_t)slab * lda)) != SL8_OK) return rc;
        if ((rc = ensure(h, &pp.d_d[i], &hd, (size_t)slab * ldd * 2)) != SL8_OK) return rc;
        if ((rc = ensure(h, &pp.d_r[i], &hr, (size_t)slab * ldr * 2)) != SL8_OK) return rc;
        if ((rc = ensure(h, &pp.d_h[i], &hh, (size_t)slab * ld_hidden)) != SL8_OK) return rc;
        if (i == HostPipe::SLOTS - 1) { pp.a_bytes = ha; pp.d_bytes = hd; pp.r_bytes = hr; pp.h_bytes = hh; }
    }
    const size_t b1 = (size_t)d_ff * ((flags & SL8_FLAG_BIAS_F32) ? 4 : 2), b2 = (size_t)d_model * ((flags & SL8_FLAG_BIAS_F32) ? 4 : 2);
    if ((rc = ensure(h, &pp.d_b, &pp.b_bytes, (size_t)d_ff * ldw1)) != SL8_OK) return rc;
    if ((rc = ensure(h, &pp.d_b2, &pp.b2_bytes, (size_t)d_model * ldw2)) != SL8_OK) return rc;
    if (bias1 && (rc = ensure(h, &pp.d_bias, &pp.bias_bytes, b1)) != SL8_OK) return rc;
    if (bias2 && (rc = ensure(h, &pp.d_bias2, &pp.bias2_bytes, b2)) != SL8_OK) return rc;

    cudaError_t e;
    auto bail = [&](cudaError_t err, const char* what) {
        cudaDeviceSynchronize();
        (void)cudaGetLastError();
        return fail_cuda(h, err, what);
    };
    cudaStream_t s0 = pp.stream[0];
    pp.h_scales[0] = scale_a; pp.h_scales[1] = scale_w1; pp.h_scales[2] = hidden_scale; pp.h_scales[3] = scale_w2;
    if ((e = cudaMemcpyAsync(pp.d_scales, pp.h_scales, 16, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of the scales");
    if ((e = cudaMemcpyAsync(pp.d_b, W1, (size_t)d_ff * ldw1, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of W1");
    if ((e = cudaMemcpyAsync(pp.d_b2, W2, (size_t)d_model * ldw2, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of W2");
    if (bias1 && (e = cudaMemcpyAsync(pp.d_bias, bias1, b1, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of bias1");
    if (bias2 && (e = cudaMemcpyAsync(pp.d_bias2, bias2, b2, cudaMemcpyHostToDevice, s0)) != cudaSuccess) return bail(e, "upload of bias2");
    if ((e = cudaEventRecord(pp.consts_ready, s0)) != cudaSuccess) return bail(e, "upload of constants");

    const uint8_t* hA = static_cast<const uint8_t*>(A);
    const uint8_t* hR = static_cast<const uint8_t*>(residual);
    uint8_t* hD = static_cast<uint8_t*>(D);
    int slot = 0;
    for (long long r0 = 0; r0 < M; r0 += slab, slot = (slot + 1) % HostPipe::SLOTS) {
        const long long rows = (r0 + slab < M) ? slab : M - r0;
        cudaStream_t s = pp.stream[slot];
        if ((slot != 0 || r0 == 0) && (e = cudaStreamWaitEvent(s, pp.consts_ready, 0)) != cudaSuccess) return bail(e, "wait for the constants");
        if ((e = cudaMemcpyAsync(pp.d_a[slot], hA + (size_t)r0 * lda, (size_t)rows * lda, cudaMemcpyHostToDevice, s)) != cudaSuccess) return bail(e, "upload of a slab of A");
        if ((e = cudaMemcpyAsync(pp.d_r[slot], hR + (size_t)r0 * ldr * 2, (size_t)rows * ldr * 2, cudaMemcpyHostToDevice, s)) != cudaSuccess) return bail(e, "upload of a slab of the residual");
        ChainArgs c = {pp.d_a[slot], lda, pp.d_b, ldw1, bias1 ? pp.d_bias : nullptr, pp.d_b2, ldw2, bias2 ? pp.d_bias2 : nullptr,
                       pp.d_r[slot], ldr, pp.d_d[slot], ldd, rows, d_model, d_ff, flags};
        rc = run_chain(h, c, pp.d_scales, pp.d_scales + 1, pp.d_scales + 3, pp.d_scales + 2, pp.d_h[slot], ld_hidden, s);
        if (rc != SL8_OK) { cudaDeviceSynchronize(); return rc; }
        if ((e = cudaMemcpyAsync(hD + (size_t)r0 * ldd * 2, pp.d_d[slot], (size_t)rows * ldd * 2, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return bail(e, "download of a slab of D");
    }
    for (int i = 0; i < HostPipe::SLOTS; i++) {
        e = cudaStreamSynchronize(pp.stream[i]);
        if (e != cudaSuccess) return fail_cuda(h, e, "host-operand pipeline");
    }
    return SL8_OK;
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
    int vid = (h && h->forced_variant >= 0) ? h->forced_variant : pick_variant(op, out_dtype, M, N, K, 0u);
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
                                  "epilogue waiting for table / residual data",
                                  "table / residual loader waiting for a free staging box"};
    constexpr unsigned kNames = sizeof names / sizeof names[0];
    snprintf(buf, sizeof buf, "device wait expired: %s (index %u, tile %u, block %u)", st[0] < kNames ? names[st[0]] : "?", st[1],
             st[2], st[3]);
    return fail(h, SL8_ERR_DEVICE_TIMEOUT, buf);
}

SL8_API int sl8_set_wait_budget_us(sl8_handle_t h, int64_t us) {
    if (!h || us < 1 || us > 4000000000ll) return SL8_ERR_INVALID_VALUE;
    h->wait_budget_us = static_cast<unsigned>(us);
    return SL8_OK;
}

SL8_API int sl8_set_wait_budget_ms(sl8_handle_t h, int ms) {
    if (ms < 1) return SL8_ERR_INVALID_VALUE;
    return sl8_set_wait_budget_us(h, static_cast<int64_t>(ms) * 1000);
}

// =========================================================================== tracing

SL8_API int sl8_trace_enable(sl8_handle_t h, int on) {
    if (!h) return SL8_ERR_INVALID_VALUE;
    std::lock_guard<std::mutex> lock(h->mu);
    DeviceGuard guard(h->device);
    h->trace_coarse = (on == 2);
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
