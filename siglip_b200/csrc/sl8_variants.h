// sl8_variants.h -- the list of compiled kernel configurations and the table entry each
// one exports.  The dispatch table in sl8_api.cu picks one entry per (layer, M, N, K); the
// reference has a single configuration fixed by compile-time macros
// (kernel_common.cuh:18-51,86-88).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "sl8_kernel.cuh"

// X(id, CG, TN, TK, STAGES, EPI_WARPS, NBUF)
//   CG         1 = one CTA per 128 x TN tile, 2 = CTA pair per 256 x TN tile
//   TK         bytes of K per pipeline stage: 128 or 256 (one or two swizzle atoms; with 256 the
//              MMA thread issues eight MMAs per barrier round trip instead of four)
//   STAGES     depth of the operand ring (bounded by the 227 KiB of shared memory)
//   EPI_WARPS  4 = one warp per TMEM lane quadrant, 8 = two (each takes half the columns), 16 = four (a quarter each;
//              e4m3 output then goes through 64-byte staging rows)
//   NBUF       staging buffers (32 rows x 128 bytes) per epilogue warp.  The layers with side data
//              (patch-embed table, FC2 residual) prefetch it NBUF - 1 regions ahead and need
//              NBUF >= 2; a variant with NBUF = 1 serves FC1 only.
#define SL8_VARIANT_LIST(X)      \
    X(0, 1, 256, 128, 3, 4, 2)   \
    X(1, 2, 256, 128, 5, 4, 3)   \
    X(2, 2, 256, 128, 5, 8, 1)   \
    X(3, 2, 256, 128, 4, 8, 2)   \
    X(4, 2, 256, 128, 5, 4, 2)   \
    X(5, 2, 256, 128, 4, 4, 4)   \
    X(6, 1, 128, 128, 5, 4, 2)   \
    X(7, 2, 128, 128, 7, 4, 2)   \
    X(8, 2, 256, 128, 6, 4, 1)   \
    X(9, 2, 256, 256, 3, 4, 1)   \
    X(10, 2, 256, 256, 2, 4, 4)  \
    X(11, 2, 256, 256, 2, 8, 2)  \
    X(12, 2, 256, 128, 3, 8, 3)  \
    X(13, 2, 256, 128, 4, 4, 3)  \
    X(14, 2, 256, 128, 4, 16, 1)  \
    X(15, 2, 256, 128, 5, 16, 1) \
    X(16, 2, 256, 128, 6, 4, 2)  \
    X(17, 2, 256, 128, 4, 8, 3)

#define SL8_NUM_VARIANTS 18

namespace sl8 {

// Kernel slots of a variant: layer x output type.
enum : int { K_PE = 0, K_FC1_BF16 = 1, K_FC1_E4M3 = 2, K_FC2 = 3, K_COUNT = 4 };

// map_bt: B with a box as tall as one CTA's share of the last, narrower N tile (== map_b when N % tile N == 0).
typedef cudaError_t (*launch_fn)(const CUtensorMap* map_a, const CUtensorMap* map_b, const CUtensorMap* map_bt,
                                 const CUtensorMap* map_d, const CUtensorMap* map_s, const KernelParams* params, int grid,
                                 cudaStream_t stream);

struct VariantEntry {
    int id;
    int cg, tn, tk, stages, epi_warps, nbuf;
    int threads;
    int smem_bytes[K_COUNT];
    const void* kernel[K_COUNT];     // for cudaFuncSetAttribute / occupancy queries; null = layer not served
    launch_fn launch[K_COUNT];
};

}  // namespace sl8

#define SL8_DECLARE_VARIANT(id, CG, TN, TK, ST, EW, NB) extern "C" const sl8::VariantEntry* sl8_variant_##id();
SL8_VARIANT_LIST(SL8_DECLARE_VARIANT)
#undef SL8_DECLARE_VARIANT
