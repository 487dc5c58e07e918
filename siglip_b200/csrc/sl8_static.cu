// sl8_static.cu -- sl8_fc1_gelu_fp8_static: the FC1 + bias + GELU layer for callers that must not
// allocate device memory.
//
// Who that is: code running inside an inference plug-in's enqueue callback, inside a latency-critical
// serving loop whose memory pool was frozen at start-up, or in a process that was handed a fixed device
// memory budget by its host application.  For them cudaMalloc is off limits (it synchronises the whole
// device, can fail long after start-up, and bypasses the host application's accounting), so they
// cannot use sl8_create, whose handle owns a cudaMalloc'ed status block, nor sl8_trace_enable.
//
// The kernels need two small pieces of global memory besides their operands: the 16-byte status block
// the bounded waits report into, and (only when tracing) 128 bytes of per-CTA cycle counters.  Here both
// live in ONE file-scope __device__ array that is part of the library image; every GPU that loads the
// library holds a copy (SL8_STATIC_SCRATCH_BYTES, about 64 KiB) until the process exits.
//
// Rules that follow from sharing one array:
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress), resolves the
//     driver's tensor-map encoder and raises the kernel's shared-memory limit.  None of that allocates,
//     but none of it belongs inside a stream capture either: make the first call before capturing.
//   * Every call on a device uses the same array, and it keeps the previous call's contents.  The status
//     block is cleared on the stream before each launch; trace records are overwritten by each traced
//     launch.  Two calls that overlap on the GPU (different streams) race on it.
//   * A launch needs one trace record per CTA; a grid of more than SL8_STATIC_MAX_CTAS CTAs is refused.
//
// Role in the whole: an additional entry point beside sl8_fc1_gelu_fp8 (sl8_api.cu); same kernel
// (variant 2 of sl8_variants.h: CTA pair, 256 x 256 tile, eight epilogue warps), same arithmetic.  It has
// no counterpart in the reference, whose hosts allocate everything in main().
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "../../include/siglip_fp8.h"
#include "sl8_variants.h"

#define SL8_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int kMaxCtas = SL8_STATIC_MAX_CTAS;
constexpr int kTraceOffset = 256;   // bytes; the status block sits at offset 0
static_assert(SL8_STATIC_SCRATCH_BYTES == kTraceOffset + SL8_STATIC_MAX_CTAS * SL8_TRACE_SLOTS * 8, "header and library disagree");
static_assert(SL8_TRACE_SLOTS == sl8::PROF_SLOTS, "header and kernel disagree");

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a
// device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_scratch[SL8_STATIC_SCRATCH_BYTES];

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    unsigned char* scratch = nullptr;   // device address of g_scratch on this device
    encode_tiled_fn encode = nullptr;
    int sm_count = 0;
    int max_clusters[sl8::K_COUNT] = {};
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int encode_2d(encode_tiled_fn enc, CUtensorMap* map, CUtensorMapDataType dt, const void* base, unsigned long long inner,
              unsigned long long outer, unsigned long long pitch_bytes, unsigned box_inner, unsigned box_outer,
              CUtensorMapL2promotion promo) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? SL8_OK
               : SL8_ERR_CUDA;
}

// Once per device, with that device current.  Allocates nothing.
int setup_device(int dev, const sl8::VariantEntry* v, DeviceState** out) {
    DeviceState& s = g_dev[dev];
    if (!s.ready) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return SL8_ERR_CUDA;
        if (prop.major != 10 || prop.minor != 0) return SL8_ERR_ARCH;
        s.sm_count = prop.multiProcessorCount;
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_scratch) != cudaSuccess || addr == nullptr) {
            (void)cudaGetLastError();
            return SL8_ERR_CUDA;
        }
        s.scratch = static_cast<unsigned char*>(addr);
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !fn)
            return SL8_ERR_CUDA;
        s.encode = reinterpret_cast<encode_tiled_fn>(fn);
        for (int slot : {static_cast<int>(sl8::K_FC1_BF16), static_cast<int>(sl8::K_FC1_E4M3)}) {
            if (cudaFuncSetAttribute(v->kernel[slot], cudaFuncAttributeMaxDynamicSharedMemorySize, v->smem_bytes[slot]) != cudaSuccess)
                return SL8_ERR_CUDA;
            int clusters = s.sm_count / v->cg;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(s.sm_count / 2 * 2), 1, 1);
            cfg.blockDim = dim3(static_cast<unsigned>(v->threads), 1, 1);
            cfg.dynamicSmemBytes = static_cast<size_t>(v->smem_bytes[slot]);
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = static_cast<unsigned>(v->cg);
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, v->kernel[slot], &cfg) == cudaSuccess && n > 0 && n < clusters) clusters = n;
            else (void)cudaGetLastError();
            s.max_clusters[slot] = clusters > 0 ? clusters : 1;
        }
        s.ready = true;
    }
    *out = &s;
    return SL8_OK;
}

}  // namespace

SL8_API int sl8_fc1_gelu_fp8_static(const void* A, int64_t lda, const void* B, int64_t ldb, const float* scale_a,
                                    const float* scale_b, const void* bias, void* D, int64_t ldd, int out_dtype,
                                    const float* out_scale, int64_t M, int N, int K, unsigned flags,
                                    unsigned* host_status, long long* host_trace, sl8_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // ---- the checks of sl8_fc1_gelu_fp8
    if (!A || !B || !D || M < 1 || N < 1 || K < 1) return SL8_ERR_INVALID_VALUE;
    if (out_dtype != SL8_OUT_BF16 && out_dtype != SL8_OUT_E4M3) return SL8_ERR_INVALID_VALUE;
    if (flags & ~static_cast<unsigned>(SL8_FLAG_BIAS_F32)) return SL8_ERR_INVALID_VALUE;
    if (M > 0x7FFFFF00ll || N % 16 != 0) return SL8_ERR_UNSUPPORTED;
    if (lda < K || ldb < K || ldd < N) return SL8_ERR_INVALID_VALUE;
    const int ob = out_dtype == SL8_OUT_BF16 ? 2 : 1;
    if (!aligned16(A) || !aligned16(B) || !aligned16(D) || (bias && !aligned16(bias)) || lda % 16 || ldb % 16 || (ldd * ob) % 16)
        return SL8_ERR_ALIGNMENT;
    // The epilogue reads each scale with one 4-byte load: a misaligned pointer would fault on the device.
    for (const float* sc : {scale_a, scale_b, out_scale})
        if (sc && (reinterpret_cast<uintptr_t>(sc) & 3u)) return SL8_ERR_ALIGNMENT;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return SL8_ERR_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return SL8_ERR_UNSUPPORTED;
    const sl8::VariantEntry* v = sl8_variant_2();
    const int slot = out_dtype == SL8_OUT_E4M3 ? sl8::K_FC1_E4M3 : sl8::K_FC1_BF16;

    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* s = nullptr;
    int rc = setup_device(dev, v, &s);
    if (rc != SL8_OK) return rc;

    const long long tiles_m = (M + 128 * v->cg - 1) / (128 * v->cg);
    const int tiles_n = (N + v->tn - 1) / v->tn;
    const long long nt = tiles_m * tiles_n;
    if (nt > 0x7FFFFFFFll) return SL8_ERR_UNSUPPORTED;
    const int clusters = nt < s->max_clusters[slot] ? static_cast<int>(nt) : s->max_clusters[slot];
    const int grid = clusters * v->cg;
    // The static scratch has room for SL8_STATIC_MAX_CTAS trace records: a larger grid does not fit.
    if (grid > kMaxCtas) return SL8_ERR_UNSUPPORTED;

    CUtensorMap map_a, map_b, map_bt, map_d;
    if ((rc = encode_2d(s->encode, &map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, (unsigned long long)K, (unsigned long long)M,
                        (unsigned long long)lda, 128, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) != SL8_OK) return rc;
    if ((rc = encode_2d(s->encode, &map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, (unsigned long long)K, (unsigned long long)N,
                        (unsigned long long)ldb, 128, (unsigned)(v->tn / v->cg), CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) != SL8_OK) return rc;
    const int tail_cols = N % v->tn == 0 ? v->tn : N % v->tn;    // the last N tile is as wide as what is left of N
    map_bt = map_b;
    if (tail_cols != v->tn &&
        (rc = encode_2d(s->encode, &map_bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, B, (unsigned long long)K, (unsigned long long)N,
                        (unsigned long long)ldb, 128, (unsigned)(tail_cols / v->cg), CU_TENSOR_MAP_L2_PROMOTION_L2_256B)) != SL8_OK) return rc;
    if ((rc = encode_2d(s->encode, &map_d, ob == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, D,
                        (unsigned long long)N, (unsigned long long)M, (unsigned long long)ldd * ob, (unsigned)(128 / ob), 32,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE)) != SL8_OK) return rc;

    sl8::KernelParams p;
    memset(&p, 0, sizeof p);
    p.M = M;
    p.N = N;
    p.K = K;
    p.tiles_n = tiles_n;
    p.num_tiles = static_cast<int>(nt);
    p.k_blocks = (K + v->tk - 1) / v->tk;
    p.last_kblock_mmas = (K - (p.k_blocks - 1) * v->tk + 31) / 32;
    p.tail_cols = tail_cols;
    p.scale_a = scale_a;
    p.scale_b = scale_b;
    p.out_scale = out_scale;
    p.bias = bias;
    p.period = 1;
    p.D = D;
    p.ldd = ldd;
    p.flags = flags;
    p.wait_budget_us = 2000000;
    p.status = reinterpret_cast<uint32_t*>(s->scratch);                               // device address, from set-up
    p.prof = host_trace ? reinterpret_cast<long long*>(s->scratch + kTraceOffset) : nullptr;

    // The array still holds the previous call's status: it has to start at zero.
    if (cudaMemsetAsync(s->scratch, 0, 16, stream) != cudaSuccess) { (void)cudaGetLastError(); return SL8_ERR_CUDA; }
    if (v->launch[slot](&map_a, &map_b, &map_bt, &map_d, &map_d, &p, grid, stream) != cudaSuccess) {
        (void)cudaGetLastError();
        return SL8_ERR_CUDA;
    }
    // From here on the kernel IS enqueued.  If one of the two read-back copies cannot be enqueued the call still
    // reports the launch (the grid size): D will be written; only host_status / host_trace stay as they were, which
    // the caller can tell from the sentinel it put there (the copies never leave word 0 of host_status at 0xFFFFFFFF).
    if (host_status && cudaMemcpyAsync(host_status, s->scratch, 16, cudaMemcpyDeviceToHost, stream) != cudaSuccess) (void)cudaGetLastError();
    if (host_trace && cudaMemcpyAsync(host_trace, s->scratch + kTraceOffset, static_cast<size_t>(grid) * SL8_TRACE_SLOTS * 8,
                                      cudaMemcpyDeviceToHost, stream) != cudaSuccess) (void)cudaGetLastError();
    return grid;   // > 0: CTAs launched = trace records that will arrive in host_trace
}
