// sl8_prep.cu -- the producer-side steps of the C ABI (include/siglip_fp8.h): what feeds the GEMMs' A operand.
#include <cuda_bf16.h>

#include "sl8_internal.h"

namespace {

inline int fail(sl8_handle_t h, int code, const std::string& msg) { return sl8_fail(h, code, msg); }
inline int fail_cuda(sl8_handle_t h, cudaError_t e, const char* what) { return sl8_fail_cuda(h, e, what); }
inline bool aligned16(const void* p) { return sl8_aligned16(p); }
typedef Sl8DeviceGuard DeviceGuard;

}  // namespace

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
