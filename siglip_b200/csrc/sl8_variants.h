// sl8_variants.h -- the list of compiled kernel configurations and the table entry each
// one exports.  The dispatch table in sl8_api.cu picks one entry per (layer, M, N, K); the
// reference has a single configuration fixed by compile-time macros
// (kernel_common.cuh:18-51,86-88).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "sl8_kernel.cuh"

// X(id, CG, TN, STAGES, EPI_WARPS, TMA_STORE)
//   CG         1 = one CTA per 128 x TN tile, 2 = CTA pair per 256 x TN tile
//   STAGES     depth of the operand ring (bounded by the 227 KiB of shared memory)
//   EPI_WARPS  4 = one warp per TMEM lane quadrant, 8 = two (each takes half the columns)
//   TMA_STORE  1 = swizzled staging + TMA tensor stores, 0 = 16-byte stores from registers
#define SL8_VARIANT_LIST(X) \
    X(0, 1, 256, 4, 4, 0)   \
    X(1, 1, 256, 3, 4, 1)   \
    X(2, 2, 256, 6, 4, 0)   \
    X(3, 2, 256, 5, 4, 1)   \
    X(4, 2, 256, 5, 8, 1)   \
    X(5, 2, 256, 6, 8, 0)   \
    X(6, 2, 192, 6, 4, 1)   \
    X(7, 2, 192, 7, 4, 0)   \
    X(8, 1, 128, 5, 4, 1)   \
    X(9, 2, 128, 7, 4, 1)   \
    X(10, 1, 256, 4, 8, 0)  \
    X(11, 2, 256, 4, 8, 1)

#define SL8_NUM_VARIANTS 12

namespace sl8 {

// Kernel slots of a variant: layer x output type.
enum : int { K_PE = 0, K_FC1_BF16 = 1, K_FC1_E4M3 = 2, K_FC2 = 3, K_COUNT = 4 };

typedef cudaError_t (*launch_fn)(const CUtensorMap* map_a, const CUtensorMap* map_b, const CUtensorMap* map_d,
                                 const KernelParams* params, int grid, cudaStream_t stream);

struct VariantEntry {
    int id;
    int cg, tn, stages, epi_warps, tma_store;
    int threads;
    int tma_store_slot[K_COUNT];     // tma_store per kernel slot (an e4m3 kernel may fall back to direct stores)
    int smem_bytes[K_COUNT];
    const void* kernel[K_COUNT];     // for cudaFuncSetAttribute / occupancy queries
    launch_fn launch[K_COUNT];
};

}  // namespace sl8

#define SL8_DECLARE_VARIANT(id, CG, TN, ST, EW, TS) extern "C" const sl8::VariantEntry* sl8_variant_##id();
SL8_VARIANT_LIST(SL8_DECLARE_VARIANT)
#undef SL8_DECLARE_VARIANT
