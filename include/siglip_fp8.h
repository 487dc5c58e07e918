/*
 * siglip_fp8.h -- C ABI of libsiglip_fp8.so
 *
 * FP8 (e4m3) GEMM engine for the three dense contractions of a SigLIP ViT
 * encoder block on NVIDIA B200 (sm_100a):
 *
 *     patch-embed : D = bf16( bf16(sa*sb * A.B^T) + table[(m + row_phase) % period, n] )
 *     FC1 + GELU  : D = cast( gelu_tanh(sa*sb * A.B^T + bias[n]) / out_scale )
 *     FC2 + res.  : D = bf16( sa*sb * A.B^T + bias[n] + residual[m, n] )
 *
 * Operand conventions are those of the reference project's per-layer launch
 * points (stephendliang/siglip):
 *     A [M, K] e4m3, K contiguous   (patch_embed.cu:159-160  tensor map dims {K, M})
 *     B [N, K] e4m3, K contiguous   (patch_embed.cu:172-173  dims {K, N}: weights stored out x in)
 *     D [M, N] bf16, N contiguous   (patch_embed.cu:187-188  dims {N, M})
 * and each sl8_* layer call replaces one of its kernel launches
 *     persistent_gemm<Op><<<148, 192, SMEM_BYTES>>>(tma_a, tma_b, tma_c, side_data, C, residual)
 * (kernel_body.cuh:448-457) together with the three cuTensorMapEncodeTiled calls
 * and the cudaFuncSetAttribute call that precede it in each layer's main().
 *
 * Differences from the reference launch, all additive:
 *   - M, N, K and the leading dimensions are run-time arguments (the reference
 *     fixes them at compile time, kernel_common.cuh:78-92);
 *   - per-tensor dequantisation scales scale_a / scale_b multiply the FP32
 *     accumulator before the epilogue (the reference consumes raw codes, i.e.
 *     scale 1); they are DEVICE pointers to one float, NULL meaning 1.0f;
 *   - FC1 can emit e4m3 directly (for the FC1 -> FC2 chain);
 *   - the positional table is a plain row-major [period, N] bf16 array (the
 *     reference wants a 32x32-blocked bias+pos table, patch_embed.cu:79-98).
 *
 * All pointers except `h`, the handle, are device pointers unless the function
 * name ends in _host.  Calls are asynchronous with respect to the host and
 * ordered on `stream` like a kernel launch.  Nothing is allocated on the call
 * path of the device-pointer entry points.
 *
 * Alignment rules (checked; violation returns SL8_ERR_ALIGNMENT):
 *   A, B, D, residual, table base addresses: 16 bytes;
 *   lda, ldb (elements = bytes): multiples of 16; ldd, ldr, ld of table in
 *   elements: such that the row pitch in bytes is a multiple of 16;
 *   N must be a multiple of 16.  K and M are arbitrary (>= 1).
 */
#ifndef SIGLIP_FP8_H_
#define SIGLIP_FP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct sl8_context* sl8_handle_t;

/* cudaStream_t without dragging the CUDA headers into C callers. */
typedef void* sl8_stream_t;

/* ---- status codes (0 = success, negative = failure); never exit(), never throw:
 * the reference's CUDA_CHECK / CU_CHECK print and exit(1) (kernel_common.cuh:123-138). */
enum {
    SL8_OK                 = 0,
    SL8_ERR_INVALID_VALUE  = -1,  /* NULL pointer, non-positive size, unknown enum            */
    SL8_ERR_ALIGNMENT      = -2,  /* base pointer or pitch breaks the 16-byte rules above      */
    SL8_ERR_UNSUPPORTED    = -3,  /* shape outside what the kernels cover (e.g. N % 16 != 0)   */
    SL8_ERR_CUDA           = -4,  /* a CUDA runtime / driver call failed; see sl8_last_error   */
    SL8_ERR_DEVICE_TIMEOUT = -5,  /* a bounded device-side wait expired (sl8_device_status)    */
    SL8_ERR_ARCH           = -6,  /* device is not compute capability 10.0                     */
    SL8_ERR_NO_DEVICE      = -7   /* no CUDA device / driver                                   */
};

/* Output element type of FC1. */
enum { SL8_OUT_BF16 = 0, SL8_OUT_E4M3 = 1 };

/* Layer ids, in the order of the reference's EpilogueOp (kernel_body.cuh:8). */
enum { SL8_OP_PATCH_EMBED = 0, SL8_OP_FC1_GELU = 1, SL8_OP_FC2_RESIDUAL = 2 };

/* Flags (bitwise or). */
enum {
    SL8_FLAG_NONE        = 0,
    /* bias is fp32 [N] as in the reference (kernel_body.cuh:12-13) instead of bf16 [N]. */
    SL8_FLAG_BIAS_F32    = 1,
    /* patch-embed: add the table in fp32 and round once, instead of the reference's
     * bf16-domain add of bf16(acc) and the table (patch_embed.cu:44-58). */
    SL8_FLAG_PE_F32_ADD  = 2,
    /* FC1 entry points: no activation, D = acc * scale + bias (what sl8_linear_bias_fp8 sets). */
    SL8_FLAG_NO_ACTIVATION = 4,
    /* FC1: GELU through the hardware tanh (tanh.approx.f32, relative error ~2^-11): one special-function operation
     * per element instead of two.  |error| <= ~2.5e-4 |x| against the exact form; off by default. */
    SL8_FLAG_GELU_HW_TANH = 8
};

/* Which kernel variant the dispatch table picks for a problem. */
typedef struct sl8_config {
    int cta_group;     /* 1 = one CTA per tile, 2 = CTA pair (tcgen05 cta_group::2)        */
    int tile_m;        /* rows per tile (128 * cta_group)                                    */
    int tile_n;        /* columns per tile                                                   */
    int tile_k;        /* K bytes per pipeline stage                                         */
    int stages;        /* depth of the TMA -> MMA shared-memory ring                          */
    int epi_warps;     /* epilogue warps per CTA                                              */
    int staging_buffers; /* swizzled staging regions per epilogue warp (1 = FC1 only)          */
    int grid;          /* CTAs launched                                                      */
    int smem_bytes;    /* dynamic shared memory per CTA                                      */
    int variant_id;    /* index usable with SL8_FORCE_VARIANT / sl8_set_variant              */
} sl8_config;

/* ---- life cycle ------------------------------------------------------------------- */

/* Creates a handle bound to CUDA device `device`.  Owns: one 16-byte device status
 * block, the dispatch table, and (only if a *_host entry point is used) pinned and
 * device staging buffers.  Replaces the per-main() setup at patch_embed.cu:104-200. */
int sl8_create(sl8_handle_t* h, int device);
int sl8_destroy(sl8_handle_t h);

/* Text of the last failure on this handle (never NULL).  With h == NULL: the last
 * failure of sl8_create on the calling thread. */
const char* sl8_last_error_string(sl8_handle_t h);

/* Library identification: "siglip_fp8 <version> sm_100a". */
const char* sl8_version(void);

/* ---- the three layers ---------------------------------------------------------------- */

/* Patch-embed GEMM + periodic table add.  Replaces persistent_gemm<BIAS_ADD>
 * (patch_embed.cu:200,216; epilogue patch_embed.cu:44-58; row -> table row
 * kernel_body.cuh:71).  `table` is bf16 [table_rows, N] with leading dimension ld_table
 * (elements); row r holds bf16(bias + pos[r % period]) as the reference's table does
 * (patch_embed.cu:79-98).  row_phase shifts the period for shards that do not start on an
 * image boundary: row m uses table row (m + row_phase) % period.
 * table_rows >= period.  Like the reference's table, which is padded to a multiple of 32 rows
 * with rows that repeat its beginning (COMB_PADDED_ROWS, patch_embed.cu:17,87), the table may
 * continue periodically past `period`; with table_rows >= period + 127 every 128-row tile of the
 * output reads one contiguous block of table rows (fast path).  A table of exactly `period` rows
 * is accepted and correct, but tiles that straddle its end are served by a slow copy loop.
 * sl8_make_periodic_table / sl8_extend_periodic_table build a padded table. */
int sl8_patch_embed_fp8(sl8_handle_t h,
                        const void* A, int64_t lda,
                        const void* B, int64_t ldb,
                        const float* scale_a, const float* scale_b,
                        const void* table, int64_t ld_table, int period, int table_rows, int row_phase,
                        void* D, int64_t ldd,
                        int64_t M, int N, int K,
                        unsigned flags, sl8_stream_t stream);

/* Counterpart of the reference's precompute_combined kernel (patch_embed.cu:79-98), row-major:
 * table[r, c] = bf16(bias[c] + pos[r % period, c]) for r < rows_out.  bias fp32 [N] (NULL = 0),
 * pos fp32 [period, N] contiguous, table bf16 with leading dimension ld_table; all device
 * pointers, caller-owned.  Use rows_out = sl8_padded_table_rows(period). */
int sl8_make_periodic_table(sl8_handle_t h, const float* bias, const float* pos, int period, int N,
                            void* table, int64_t ld_table, int rows_out, sl8_stream_t stream);

/* Same for a table that already exists in bf16: out[r] = in[r % period], r < rows_out. */
int sl8_extend_periodic_table(sl8_handle_t h, const void* table_in, int64_t ld_in, int period, int N,
                              void* table_out, int64_t ld_out, int rows_out, sl8_stream_t stream);

/* period + 127 rounded up to a multiple of 32: the row count of a padded table. */
int sl8_padded_table_rows(int period);

/* FC1 GEMM + bias + GELU(tanh).  Replaces persistent_gemm<BIAS_GELU>
 * (fc1_gelu.cu:131,147; gelu_fwd fc1_gelu.cu:16-19).  out_dtype SL8_OUT_BF16 writes
 * bf16(g); SL8_OUT_E4M3 writes e4m3_sat_rne(g * (1 / *out_scale)), out_scale a device
 * pointer to one float (NULL = 1).  ldd is in elements of the output type. */
int sl8_fc1_gelu_fp8(sl8_handle_t h,
                     const void* A, int64_t lda,
                     const void* B, int64_t ldb,
                     const float* scale_a, const float* scale_b,
                     const void* bias,
                     void* D, int64_t ldd, int out_dtype, const float* out_scale,
                     int64_t M, int N, int K,
                     unsigned flags, sl8_stream_t stream);

/* GEMM + bias with no activation: the block's Q, K, V projections (the reference lists them as the next
 * GEMMs of the block, docs/architecture.md:76-90, and has no kernel for them; the output projection, bias +
 * residual, is sl8_fc2_residual_fp8).  Same kernels, arguments and output types as sl8_fc1_gelu_fp8, of which
 * this is the SL8_FLAG_NO_ACTIVATION form: D = bf16(acc * scale_a * scale_b + bias) or its e4m3 quantisation. */
int sl8_linear_bias_fp8(sl8_handle_t h,
                        const void* A, int64_t lda,
                        const void* B, int64_t ldb,
                        const float* scale_a, const float* scale_b,
                        const void* bias,
                        void* D, int64_t ldd, int out_dtype, const float* out_scale,
                        int64_t M, int N, int K,
                        unsigned flags, sl8_stream_t stream);

/* FC2 GEMM + bias + residual.  Replaces persistent_gemm<BIAS_RESIDUAL>
 * (fc2.cu:162,178; epilogue fc2.cu:19-54): D = bf16((acc + bias) + float(residual)). */
int sl8_fc2_residual_fp8(sl8_handle_t h,
                         const void* A, int64_t lda,
                         const void* B, int64_t ldb,
                         const float* scale_a, const float* scale_b,
                         const void* bias,
                         const void* residual, int64_t ldr,
                         void* D, int64_t ldd,
                         int64_t M, int N, int K,
                         unsigned flags, sl8_stream_t stream);

/* ---- producer-side steps: what feeds A ---------------------------------------------------
 * No counterpart in the reference, which starts at the GEMM operands (its docs describe the patch embedding as
 * "Conv2d as GEMM", docs/architecture.md:11-12, and leave the unfold and the quantisation to the caller). */
enum { SL8_DT_F32 = 0, SL8_DT_BF16 = 1 };

/* Patch unfold fused with the per-tensor quantisation: pixels [images, channels, height, width] (contiguous, fp32
 * or bf16) -> A [images * gh * gw, channels * patch * patch] e4m3 with row pitch lda, gh = height / patch,
 * gw = width / patch (pixels past gh * patch, gw * patch are not used).  Row (img * gh + gy) * gw + gx, column
 * c * patch^2 + py * patch + px -- the flattening of a Conv2d weight [N, C, patch, patch] -- holds
 * e4m3_sat_rne(pixel * (1 / *scale)); scale is a device pointer to the activation scale the GEMM is given as scale_a
 * (NULL = 1).  The pad columns up to lda are written as zeros when lda - K < 128. */
int sl8_patchify_quantize_e4m3(sl8_handle_t h, const void* pixels, int pixel_dtype, int images, int channels,
                               int height, int width, int patch, const float* scale,
                               void* A, int64_t lda, sl8_stream_t stream);

/* Dynamic per-tensor scale of an activation x [rows, cols] (fp32 or bf16, leading dimension ld elements):
 * *amax = max |x| and, if scale is not NULL, *scale = amax / 448 (1 for an all-zero tensor).  Device pointers. */
int sl8_amax_scale(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld,
                   float* amax, float* scale, sl8_stream_t stream);

/* out[r, c] = e4m3_sat_rne(x[r, c] * (1 / *scale)): the quantisation FC1 fuses when it is given a static out_scale,
 * as a separate pass for a scale that sl8_amax_scale has just produced. */
int sl8_quantize_e4m3(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld,
                      const float* scale, void* out, int64_t ld_out, sl8_stream_t stream);

/* LayerNorm fused with the quantisation of its output: FC1's A operand straight from the residual stream (the
 * reference lists this fusion as unstarted, docs/architecture.md:92-101).  x [rows, cols] fp32 or bf16, gamma / beta
 * fp32 [cols] (NULL = 1 / 0), statistics in fp32 over the row, out[r, c] = e4m3_sat_rne(((x - mean) * rsqrt(var + eps)
 * * gamma + beta) * (1 / *scale)).  cols, ld and ld_out must be multiples of 8. */
int sl8_layernorm_quantize_e4m3(sl8_handle_t h, const void* x, int dtype, int64_t rows, int cols, int64_t ld,
                                const float* gamma, const float* beta, float eps, const float* scale,
                                void* out, int64_t ld_out, sl8_stream_t stream);

/* ---- the same three layers with HOST operands ------------------------------------------
 * What each reference main() does around its launch (upload operands, launch, download
 * all of C: patch_embed.cu:111-154,249-252), as one call: rows are cut into slabs that
 * are uploaded, computed and downloaded on three streams so the copies overlap the
 * kernels.  A, residual and D are host pointers (pinned memory gives full PCIe speed);
 * B, bias, table and the scale/out_scale VALUES are host data too and are uploaded once
 * per call.  Blocking: returns when D is complete in host memory.  Staging buffers are
 * allocated by the handle on first use and kept. */
int sl8_patch_embed_fp8_host(sl8_handle_t h,
                             const void* A, int64_t lda, const void* B, int64_t ldb,
                             float scale_a, float scale_b,
                             const void* table, int64_t ld_table, int period, int table_rows, int row_phase,
                             void* D, int64_t ldd, int64_t M, int N, int K, unsigned flags);
int sl8_fc1_gelu_fp8_host(sl8_handle_t h,
                          const void* A, int64_t lda, const void* B, int64_t ldb,
                          float scale_a, float scale_b, const void* bias,
                          void* D, int64_t ldd, int out_dtype, float out_scale,
                          int64_t M, int N, int K, unsigned flags);
int sl8_fc2_residual_fp8_host(sl8_handle_t h,
                              const void* A, int64_t lda, const void* B, int64_t ldb,
                              float scale_a, float scale_b, const void* bias,
                              const void* residual, int64_t ldr,
                              void* D, int64_t ldd, int64_t M, int N, int K, unsigned flags);

/* ---- the MLP of the block as one call: FC1 + GELU -> e4m3 -> FC2 + residual ---------------------------------
 * The reference runs the two layers as two programs (fc1_gelu.cu, fc2.cu) and lists their hand-over as open work
 * (docs/architecture.md:92-101); here FC1 writes e4m3 codes with a static scale straight into FC2's operand.
 *   hidden = e4m3_sat_rne( gelu_tanh(sa*sw1 * A.W1^T + bias1) / *hidden_scale )      [M, d_ff], row pitch ld_hidden
 *   D      = bf16( (*hidden_scale)*sw2 * hidden.W2^T + bias2 + residual )             [M, d_model]
 * A [M, d_model] e4m3, W1 [d_ff, d_model] e4m3, W2 [d_model, d_ff] e4m3, biases bf16 (fp32 with SL8_FLAG_BIAS_F32),
 * residual and D bf16 [M, d_model].  `hidden` is caller-owned scratch of M x ld_hidden bytes (ld_hidden >= d_ff, a
 * multiple of 16; 128 recommended); hidden_scale must not be NULL.  Both launches go to `stream`; flags:
 * SL8_FLAG_BIAS_F32, SL8_FLAG_GELU_HW_TANH.  Equivalent to sl8_fc1_gelu_fp8(..., SL8_OUT_E4M3, hidden_scale) followed
 * by sl8_fc2_residual_fp8(hidden, ..., scale_a = hidden_scale). */
int sl8_mlp_chain_fp8(sl8_handle_t h,
                      const void* A, int64_t lda,
                      const void* W1, int64_t ldw1, const float* scale_a, const float* scale_w1, const void* bias1,
                      void* hidden, int64_t ld_hidden, const float* hidden_scale,
                      const void* W2, int64_t ldw2, const float* scale_w2, const void* bias2,
                      const void* residual, int64_t ldr,
                      void* D, int64_t ldd,
                      int64_t M, int d_model, int d_ff,
                      unsigned flags, sl8_stream_t stream);

/* The same with HOST operands: A and the residual go up, D comes down, slab by slab on three streams; the hidden
 * activations never leave the GPU (handle-owned slabs), so a row costs d_model + 4 * d_model bytes over the bus instead
 * of the d_model + 2 * d_ff (+ d_ff + 4 * d_model) of two separate *_host calls.  Scales are host values.  Blocking. */
int sl8_mlp_chain_fp8_host(sl8_handle_t h,
                           const void* A, int64_t lda,
                           const void* W1, int64_t ldw1, float scale_a, float scale_w1, const void* bias1,
                           float hidden_scale,
                           const void* W2, int64_t ldw2, float scale_w2, const void* bias2,
                           const void* residual, int64_t ldr,
                           void* D, int64_t ldd,
                           int64_t M, int d_model, int d_ff, unsigned flags);

/* ---- dispatch ------------------------------------------------------------------------- */

/* Variant the dispatch table selects for (op, out_dtype, M, N, K) and flags = 0; the reference has a
 * single compile-time configuration (kernel_common.cuh:18-51,86-88).  An FC1 call with SL8_FLAG_NO_ACTIVATION or
 * SL8_FLAG_GELU_HW_TANH runs the eight-epilogue-warp variant where this answers with a sixteen-warp one. */
int sl8_query_config(sl8_handle_t h, int op, int out_dtype, int64_t M, int N, int K, sl8_config* out);

/* Number of compiled variants, and the description of variant `variant_id`. */
int sl8_num_variants(void);
int sl8_describe_variant(int variant_id, sl8_config* out);

/* Forces every later call on this handle to use `variant_id` (-1 restores the table).
 * The environment variable SL8_FORCE_VARIANT does the same for new handles. */
int sl8_set_variant(sl8_handle_t h, int variant_id);

/* ---- device-side wait watchdog -------------------------------------------------------- */

/* Every wait inside the kernels (mbarrier polls) is bounded; a wait that expires records
 * a code in the handle's device status block and the kernel unwinds and exits normally
 * (the reference's mbar_wait spins for ever, kernel_common.cuh:166-178).
 * sl8_device_status synchronises `stream`, reads the block, clears it, and returns SL8_OK
 * or SL8_ERR_DEVICE_TIMEOUT; *detail (optional) receives role, barrier and tile of
 * the first wait that expired. */
int sl8_device_status(sl8_handle_t h, sl8_stream_t stream, unsigned detail[4]);

/* Wait budget for later launches on this handle, in milliseconds or microseconds (default 2 s).  A wait that
 * parks its thread is checked against the budget about every 0.3 ms, a spinning one every few microseconds; in a CTA
 * pair the CTA whose wait ran out tells its partner, so both leave at once. */
int sl8_set_wait_budget_ms(sl8_handle_t h, int ms);
int sl8_set_wait_budget_us(sl8_handle_t h, int64_t us);

/* ---- in-kernel tracing ------------------------------------------------------------------
 * Counterpart of the reference's -DTIMING build (clock64 stamps in the MMA thread and the
 * epilogue warps, kernel_body.cuh:523-537,569-636,695-750; host read-back print_timing
 * kernel_body.cuh:821-1001), switchable at run time instead of by recompiling.
 * sl8_trace_enable(h, 1) allocates a device buffer (the one allocation outside sl8_create;
 * not on the call path of a layer); later launches on the handle then record, per CTA,
 * SL8_TRACE_SLOTS clock-cycle totals of the LAST launch:
 *   [0] TMA producer waiting for a free stage   [1] producer total
 *   [2] MMA thread waiting for operands         [3] MMA thread waiting for a free accumulator
 *   [4] MMA thread total                        [5] epilogue warp 0 waiting for an accumulator
 *   [6] epilogue warp 0 total                   [7] epilogue warp 0 waiting for staging to drain
 *   [8] tiles of this CTA pair                  [9] epilogue warp 0 waiting for tcgen05.ld
 *   [10] epilogue warp 0 transform + staging    [11] epilogue warp 0 proxy fence + store issue
 *   [12] epilogue warp 0 waiting until the previous store has read its staging buffer
 *   [13] epilogue warp 0 issuing the side-data prefetch
 *   [14] MMA thread issuing tcgen05.mma         [15] MMA thread issuing tcgen05.commit
 * sl8_trace_enable(h, 2) records the totals and the once-per-tile waits only ([1], [3], [4], [5], [6], [8]; [2] then counts the k-blocks
 * whose operands had not landed one k-block ahead): the roles then run the same code paths as
 * without tracing, so [4] is the kernel's duration in SM clock cycles (divide by the event time for the SM clock).
 * sl8_trace_read synchronises the device and copies min(grid of the last launch, max_blocks)
 * records into out[max_blocks * SL8_TRACE_SLOTS]; returns the number of records or an error. */
#define SL8_TRACE_SLOTS 16
int sl8_trace_enable(sl8_handle_t h, int on);
int sl8_trace_read(sl8_handle_t h, long long* out, int max_blocks);

/* ---- FC1 without any device allocation ---------------------------------------------------
 * No counterpart in the reference (its hosts allocate every buffer in main()).
 *
 * For callers that are not allowed to allocate device memory -- a plug-in's enqueue callback, a
 * serving loop whose memory pool was frozen at start-up, a process living inside a fixed device
 * memory budget -- and therefore cannot call sl8_create (its handle owns a cudaMalloc'ed status
 * block) or sl8_trace_enable.  Same kernel and arithmetic as sl8_fc1_gelu_fp8; the status block and
 * the trace records live in a __device__ array inside the library image instead
 * (SL8_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process exits).
 * The call allocates nothing and needs no handle; it runs on the CURRENT device.
 *
 *   host_status  optional, 4 words of host memory: receives the status block (word 0 != 0: a device
 *                wait expired; see sl8_device_status) by a copy enqueued on `stream` after the kernel;
 *   host_trace   optional, room for SL8_TRACE_SLOTS x (return value) 64-bit counters: switches
 *                tracing on for this launch and receives one record per CTA the same way.
 * Both are valid once `stream` has been synchronised.
 *
 * Returns the number of CTAs launched (> 0) or a negative status code.  A launch of more than
 * SL8_STATIC_MAX_CTAS CTAs does not fit the scratch and is refused with SL8_ERR_UNSUPPORTED; flags
 * other than SL8_FLAG_BIAS_F32 are refused with SL8_ERR_INVALID_VALUE.
 *
 * All calls on one GPU share the one array, which keeps what the previous call left in it: the status
 * block is cleared on `stream` before every launch, and calls that overlap on the GPU (different
 * streams) race on it -- keep them on one stream.  The first call on a device looks up the array's
 * device address and prepares the kernel (no allocation); make that first call before any stream
 * capture begins. */
#define SL8_STATIC_MAX_CTAS 512
#define SL8_STATIC_SCRATCH_BYTES (256 + SL8_STATIC_MAX_CTAS * SL8_TRACE_SLOTS * 8)
int sl8_fc1_gelu_fp8_static(const void* A, int64_t lda, const void* B, int64_t ldb,
                            const float* scale_a, const float* scale_b, const void* bias,
                            void* D, int64_t ldd, int out_dtype, const float* out_scale,
                            int64_t M, int N, int K, unsigned flags,
                            unsigned* host_status, long long* host_trace, sl8_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SIGLIP_FP8_H_ */
