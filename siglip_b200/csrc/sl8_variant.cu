// sl8_variant.cu -- instantiates the four kernels (patch-embed, FC1 -> bf16, FC1 -> e4m3,
// FC2) of ONE tile configuration and exports its table entry.  Compiled once per entry of
// SL8_VARIANT_LIST with -DSL8_VARIANT_ID=<id>, so the configurations build in parallel.
#include <type_traits>

#include "sl8_variants.h"

#ifndef SL8_VARIANT_ID
#error "compile with -DSL8_VARIANT_ID=<id from SL8_VARIANT_LIST>"
#endif

namespace sl8 {
namespace {

template <int CG, int TN, int TK, int STAGES, int EW, int OP, int OUT, int NBUF>
cudaError_t launch_one(const CUtensorMap* map_a, const CUtensorMap* map_b, const CUtensorMap* map_bt, const CUtensorMap* map_d,
                       const CUtensorMap* map_s, const KernelParams* params, int grid, cudaStream_t stream) {
    using T = KernelTraits<CG, TN, TK, STAGES, EW, OUT, NBUF>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(T::THREADS, 1, 1);
    cfg.dynamicSmemBytes = T::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sl8_gemm_kernel<CG, TN, TK, STAGES, EW, OP, OUT, NBUF>, *map_a, *map_b, *map_bt, *map_d, *map_s, *params);
}

// Kernel pointer / launcher of one layer, or nulls where the variant cannot serve it.
template <int CG, int TN, int TK, int STAGES, int EW, int OP, int OUT, int NBUF, bool SERVED>
struct Slot {
    static const void* kernel() { return reinterpret_cast<const void*>(&sl8_gemm_kernel<CG, TN, TK, STAGES, EW, OP, OUT, NBUF>); }
    static launch_fn launcher() { return &launch_one<CG, TN, TK, STAGES, EW, OP, OUT, NBUF>; }
};
template <int CG, int TN, int TK, int STAGES, int EW, int OP, int OUT, int NBUF>
struct Slot<CG, TN, TK, STAGES, EW, OP, OUT, NBUF, false> {
    static const void* kernel() { return nullptr; }
    static launch_fn launcher() { return nullptr; }
};

template <int ID, int CG, int TN, int TK, int STAGES, int EW, int NBUF>
const VariantEntry* make_entry() {
    constexpr bool SIDE = NBUF >= 2;   // layers with side data need a second staging buffer
    using T16 = KernelTraits<CG, TN, TK, STAGES, EW, OUT_BF16, NBUF>;
    constexpr bool E4 = (TN / (EW / 4)) % 64 == 0;   // an e4m3 staging region is 128 or 64 columns wide
    using T8 = std::conditional_t<E4, KernelTraits<CG, TN, TK, STAGES, EW, E4 ? OUT_E4M3 : OUT_BF16, NBUF>, T16>;
    static const VariantEntry e = {
        ID, CG, TN, TK, STAGES, EW, NBUF, T16::THREADS,
        {T16::SMEM_BYTES, T16::SMEM_BYTES, T8::SMEM_BYTES, T16::SMEM_BYTES},
        {Slot<CG, TN, TK, STAGES, EW, OP_PE, OUT_BF16, NBUF, SIDE>::kernel(), Slot<CG, TN, TK, STAGES, EW, OP_FC1, OUT_BF16, NBUF, true>::kernel(),
         Slot<CG, TN, TK, STAGES, EW, OP_FC1, OUT_E4M3, NBUF, E4>::kernel(), Slot<CG, TN, TK, STAGES, EW, OP_FC2, OUT_BF16, NBUF, SIDE>::kernel()},
        {Slot<CG, TN, TK, STAGES, EW, OP_PE, OUT_BF16, NBUF, SIDE>::launcher(), Slot<CG, TN, TK, STAGES, EW, OP_FC1, OUT_BF16, NBUF, true>::launcher(),
         Slot<CG, TN, TK, STAGES, EW, OP_FC1, OUT_E4M3, NBUF, E4>::launcher(), Slot<CG, TN, TK, STAGES, EW, OP_FC2, OUT_BF16, NBUF, SIDE>::launcher()}};
    return &e;
}

}  // namespace
}  // namespace sl8

#define SL8_CAT2(a, b) a##b
#define SL8_CAT(a, b) SL8_CAT2(a, b)

#define SL8_DEFINE_IF_SELECTED(id, CG, TN, TK, ST, EW, NB)                                     \
    template <int SEL, typename = void>                                                    \
    struct SL8_CAT(Pick, id) {                                                             \
        static const sl8::VariantEntry* get() { return nullptr; }                          \
    };                                                                                     \
    template <typename V>                                                                  \
    struct SL8_CAT(Pick, id)<id, V> {                                                      \
        static const sl8::VariantEntry* get() { return sl8::make_entry<id, CG, TN, TK, ST, EW, NB>(); } \
    };
SL8_VARIANT_LIST(SL8_DEFINE_IF_SELECTED)
#undef SL8_DEFINE_IF_SELECTED

// Only the Pick<id> specialisation matching SL8_VARIANT_ID is ever instantiated, so only its
// kernels are compiled into this object.
#define SL8_ENTRY_NAME SL8_CAT(sl8_variant_, SL8_VARIANT_ID)
#define SL8_PICK_NAME SL8_CAT(Pick, SL8_VARIANT_ID)

extern "C" const sl8::VariantEntry* SL8_ENTRY_NAME() { return SL8_PICK_NAME<SL8_VARIANT_ID>::get(); }
