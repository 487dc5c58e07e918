// ref_shim.cu -- lets tests and the side-by-side bench launch the REFERENCE's own kernels on
// caller-supplied device buffers.
//
// TEST INFRASTRUCTURE ONLY; never linked into libsiglip_fp8.so.  This file contains no
// reference code: it #includes one of the reference's layer sources from where it lies
// (-I<reference checkout>, see oracle/Makefile; its main() is renamed out of the way) and adds a
// C entry point that encodes the three tensor maps the way each reference main() does
// (A {K, M} box {128,128}, B {K, N} box {128,128}, C {N, M} bf16 box {64,32}, all SWIZZLE_128B:
// patch_embed.cu:157-198) and issues the reference's launch
// persistent_gemm<Op><<<148, THREADS, SMEM_BYTES>>>(...) (patch_embed.cu:216, fc1_gelu.cu:147,
// fc2.cu:178).  The reference's shapes are compile-time constants: M = 928 256 and the N, K of
// the included layer; sl8_ref_shape reports them.
//
// SL8_REF_LAYER: 0 = patch_embed.cu, 1 = fc1_gelu.cu, 2 = fc2.cu.
#define main sl8_ref_unused_main
#if SL8_REF_LAYER == 0
#include "patch_embed.cu"
#define SL8_REF_OP EpilogueOp::BIAS_ADD
#elif SL8_REF_LAYER == 1
#include "fc1_gelu.cu"
#define SL8_REF_OP EpilogueOp::BIAS_GELU
#elif SL8_REF_LAYER == 2
#include "fc2.cu"
#define SL8_REF_OP EpilogueOp::BIAS_RESIDUAL
#else
#error "SL8_REF_LAYER must be 0, 1 or 2"
#endif
#undef main

#define SL8_REF_API extern "C" __attribute__((visibility("default")))

// M, N, K, period (SEQ_LEN) and padded table rows of the compiled reference layer.
SL8_REF_API void sl8_ref_shape(long long* m, int* n, int* k, int* seq_len, int* table_rows) {
    *m = M_TOTAL;
    *n = N_DIM;
    *k = K_DIM;
    *seq_len = SEQ_LEN;
#if SL8_REF_LAYER == 0
    *table_rows = COMB_PADDED_ROWS;
#else
    *table_rows = 0;
#endif
}

static int encode(CUtensorMap* map, CUtensorMapDataType dt, void* base, unsigned long long inner,
                  unsigned long long outer, unsigned long long pitch, unsigned box_inner, unsigned box_outer) {
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = cuTensorMapEncodeTiled(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}

// side: layer 0 = the blocked bf16 bias+pos table made by sl8_ref_make_table; layers 1, 2 = fp32 bias [N].
// residual: bf16 [M, N] for layer 2, ignored otherwise.  Returns 0 or a negative CUDA error.
SL8_REF_API int sl8_ref_launch(const void* A, const void* B, const void* side, void* C, const void* residual,
                               void* stream) {
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(persistent_gemm<SL8_REF_OP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES);
        if (e != cudaSuccess) return -(int)e;
        attr = true;
    }
    CUtensorMap ta, tb, tc;
    int rc;
    if ((rc = encode(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, const_cast<void*>(A), K_DIM, M_TOTAL, K_DIM, TK, TM))) return rc;
    if ((rc = encode(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, const_cast<void*>(B), K_DIM, N_DIM, K_DIM, TK, TN / 2))) return rc;
    if ((rc = encode(&tc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, C, N_DIM, M_TOTAL, (unsigned long long)N_DIM * 2, 64, 32))) return rc;
    persistent_gemm<SL8_REF_OP><<<SM_COUNT, THREADS, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(
        ta, tb, tc, static_cast<SideDataPtr<SL8_REF_OP>>(side), static_cast<__nv_bfloat16*>(C),
        static_cast<const __nv_bfloat16*>(residual));
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -(int)e;
}

#if SL8_REF_LAYER == 0
// Runs the reference's precompute_combined (patch_embed.cu:79-98): fp32 bias [N] and fp32 pos
// [SEQ_LEN, N] -> blocked bf16 table of COMB_PADDED_ROWS x N elements.
SL8_REF_API int sl8_ref_make_table(const float* bias, const float* pos, void* combined, void* stream) {
    const int total = COMB_PADDED_ROWS * N_DIM;
    precompute_combined<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        bias, pos, static_cast<__nv_bfloat16*>(combined), SEQ_LEN, N_DIM);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -(int)e;
}
#endif
