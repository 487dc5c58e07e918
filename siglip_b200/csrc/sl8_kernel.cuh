// sl8_kernel.cuh -- the persistent, warp-specialised FP8 GEMM kernel with fused epilogues.
//
// One kernel template covers the three layers (patch-embed + periodic table add,
// FC1 + bias + GELU, FC2 + bias + residual) and every tile configuration.  It is the
// counterpart of the reference's persistent_gemm<EpilogueOp> (kernel_body.cuh:448-815) and
// epilogue_store (kernel_body.cuh:47-442), rebuilt around run-time M/N/K:
//
//   warp 0        TMA producer of A: streams A[128 x 128B] k-blocks into a ring of STAGES
//                 shared-memory stages (SWIZZLE_128B), one mbarrier pair (full / empty) per stage,
//                 and announces the stage's bytes.
//   warp 3 + EPI  TMA producer of B: streams B[TN/CG x 128B] k-blocks into the same stages.  Two
//                 issuing threads because a thread's next bulk-tensor copy is not accepted before the
//                 TMA unit has generated the requests of its previous one (2 cycles per 128-byte row:
//                 64 bytes per clock per issuing thread, measured), while the unit itself serves two
//                 threads at once at 128 bytes per clock: one thread cannot feed a 256 x 256 tile.
//   warp 1        allocates tensor memory; one thread of the leader CTA issues
//                 tcgen05.mma kind::f8f6f4 (E4M3 x E4M3 -> FP32 in TMEM), four K=32 steps per
//                 k-block (fewer in the K tail), and commits to the stage's empty barrier and,
//                 after the last k-block, to the accumulator's full barrier.
//   warps 2..     epilogue: tcgen05.ld of the finished accumulator (two accumulators in TMEM,
//                 so the MMA of tile i+1 overlaps the epilogue of tile i), dequantisation
//                 scale, fused bias / GELU / residual / table add, conversion to bf16 or
//                 e4m3 into swizzled shared staging, TMA tensor stores.  The residual / table
//                 values of a 32-row x 128-byte region are brought into that same staging buffer
//                 by a TMA load a few regions ahead, added in place and stored from there.
//
//   last warp     side-data loader (patch-embed, FC2): one lane issues the TMA loads that bring the table /
//                 residual regions into the epilogue warps' staging buffers as those become free, so
//                 the epilogue warps never wait for a TMA instruction to be accepted.
//
// CG == 2 runs a CTA pair per tile (cluster of two, tcgen05 cta_group::2): each CTA loads its
// own 128 rows of A and half of the tile's B rows, the leader issues 256 x TN MMAs that read
// both CTAs' shared memory and write both CTAs' tensor memory.
//
// Tiles are dealt round-robin (tile = cluster index + i * clusters) in N-fastest order, so
// the clusters running at any moment share a few A row-blocks and the whole of B in L2.
//
// Every wait is bounded: when a poll loop exceeds the budget it records where it was in the
// status block, raises a CTA-wide abort flag that every other wait loop checks, and all
// roles fall through to the common exit, which still frees tensor memory.
#pragma once

#include "sl8_ptx.cuh"

#ifndef SL8_SPIN_CRITICAL
#define SL8_SPIN_CRITICAL true
#endif

namespace sl8 {

enum : int { OP_PE = 0, OP_FC1 = 1, OP_FC2 = 2 };
enum : int { OUT_BF16 = 0, OUT_E4M3 = 1 };
// Measurement aids (skip one part of the kernel to time the rest).  They cost instructions in the
// hot loops, so they exist only in a library built with -DSL8_DIAG.
#ifdef SL8_DIAG
#define SL8_DBG(flags, bit) (((flags) & (bit)) != 0u)
#else
#define SL8_DBG(flags, bit) false
#endif

// FLAG_COARSE_TRACE (set by the library, never by a caller): with tracing on, record only the per-role totals; the
// roles then run their untimed code paths, so the totals are those of the kernel as it runs without tracing.
enum : unsigned { FLAG_BIAS_F32 = 1u, FLAG_PE_F32_ADD = 2u, FLAG_NO_ACTIVATION = 4u, FLAG_GELU_HW_TANH = 8u,
                  FLAG_COARSE_TRACE = 0x40000000u,
                  FLAG_TEST_DROP_B = 0x10000000u,  // test aid (set by the library from SL8_TEST_DROP_B): the B copy of k-block 1 of each cluster's first tile is
                                                   // never issued, so the MMA thread's bounded wait for that stage runs out
                  FLAG_SINGLE_ACC = 0x20000000u,   // measurement aid (set by the library from SL8_SINGLE_ACC): one accumulator, no MMA / epilogue overlap
                  DBG_SKIP_SIDE = 0x100u, DBG_SKIP_GELU = 0x200u, DBG_SKIP_BIAS = 0x400u, DBG_SKIP_STORE = 0x800u,
                  DBG_SKIP_LOAD = 0x1000u, DBG_SKIP_EPILOGUE = 0x2000u, DBG_SKIP_MMA = 0x4000u,
                  DBG_SKIP_A = 0x8000u, DBG_SKIP_B = 0x10000u, DBG_SKIP_TMEM_LD = 0x20000u, DBG_SKIP_MATH = 0x40000u,
                  DBG_COARSE_TRACE = 0x80000000u };   // record per-role totals only (the inner timers cost ~35 cycles each)

// status[0] codes: which role gave up.
enum : uint32_t {
    ST_OK = 0,
    ST_PRODUCER_EMPTY_WAIT = 1,
    ST_MMA_FULL_WAIT = 2,
    ST_MMA_TMEM_EMPTY_WAIT = 3,
    ST_EPI_TMEM_FULL_WAIT = 4,
    ST_EPI_SIDE_WAIT = 5,
    ST_SIDE_LOADER_WAIT = 6
};

// Tracing slots written per CTA when KernelParams::prof is set (cycles, clock64).
enum : int {
    PROF_PRODUCER_WAIT = 0,   // TMA producer waiting for a free stage
    PROF_PRODUCER_TOTAL = 1,
    PROF_MMA_WAIT_FULL = 2,   // MMA thread waiting for operands
    PROF_MMA_WAIT_TMEM = 3,   // MMA thread waiting for a free accumulator
    PROF_MMA_TOTAL = 4,
    PROF_EPI_WAIT_ACC = 5,    // epilogue warp 0 waiting for a finished accumulator
    PROF_EPI_TOTAL = 6,
    PROF_EPI_WAIT_STORE = 7,  // epilogue warp 0 waiting for staging to drain
    PROF_TILES = 8,
    PROF_EPI_WAIT_LD = 9,     // epilogue warp 0 waiting for tcgen05.ld
    PROF_EPI_MATH = 10,       // epilogue warp 0: transform + staging writes
    PROF_EPI_STORE_ISSUE = 11,// epilogue warp 0: proxy fence + TMA store issue
    PROF_EPI_REFILL = 12,     // epilogue warp 0: waiting until the previous store has read its staging buffer
    PROF_EPI_PREFETCH = 13,   // epilogue warp 0: issuing the side-data prefetch
    PROF_MMA_ISSUE = 14,      // MMA thread: issuing tcgen05.mma
    PROF_MMA_COMMIT = 15,     // MMA thread: issuing tcgen05.commit
    PROF_SLOTS = 16
};

struct KernelParams {
    long long M;
    int N;
    int K;
    int tiles_n;
    int num_tiles;
    int k_blocks;          // ceil(K / TILE_K)
    int last_kblock_mmas;  // K = 32 steps needed in the last k-block (1 .. TILE_K / 32)
    int tail_cols;         // columns of the last N tile: N - (tiles_n - 1) * TN, a multiple of 16 (== TN when N % TN == 0)
    const float* scale_a;
    const float* scale_b;
    const float* out_scale;
    const void* bias;                // bf16 [N] or fp32 [N] (FLAG_BIAS_F32); may be null
    const __nv_bfloat16* side;       // table [period, N] (patch-embed) or residual [M, N] (FC2)
    long long ld_side;               // elements
    int period;
    int row_phase;
    int table_rows;                  // rows the table holds: >= period; rows past period repeat it (patch-embed)
    void* D;
    long long ldd;                   // elements of the output type
    unsigned flags;
    unsigned wait_budget_us;         // budget of every device-side wait, microseconds
    uint32_t* status;                // 4 words: code, barrier/stage, tile, block
    long long* prof;                 // optional: PROF_SLOTS clock64 totals per CTA (null = tracing off)
};

template <int CG, int TN, int TK, int STAGES, int EPI_WARPS, int OUT, int NBUF>
struct KernelTraits {
    static_assert(CG == 1 || CG == 2, "one CTA or a CTA pair per tile");
    static_assert(TN == 128 || TN == 256, "tile N");
    static_assert(EPI_WARPS == 4 || EPI_WARPS == 8 || EPI_WARPS == 16, "one, two or four warps per TMEM lane quadrant");
    static_assert(NBUF >= 1 && NBUF <= 4, "staging buffers per epilogue warp");
    static constexpr int TILE_M_CTA = 128;                       // rows per CTA = TMEM lanes
    static_assert(TK == 128 || TK == 256, "bytes of K per stage: one or two 128-byte swizzle atoms");
    static constexpr int TILE_K = TK;                            // bytes of K per stage
    static constexpr int KATOMS = TK / 128;                      // 128-byte swizzle atoms per stage and operand
    static constexpr int B_ROWS = TN / CG;                       // B rows this CTA loads per stage
    static constexpr int A_ATOM_BYTES = TILE_M_CTA * 128;        // 16 KiB: 128 rows x 128 bytes
    static constexpr int B_ATOM_BYTES = B_ROWS * 128;
    static constexpr int A_BYTES = KATOMS * A_ATOM_BYTES;
    static constexpr int B_BYTES = KATOMS * B_ATOM_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;        // also the bytes one CTA's TMA adds per stage
    static constexpr int ACC_STRIDE = TN;                        // TMEM columns between the two accumulators
    static constexpr int TMEM_COLS = 2 * TN;                     // 256 or 512: a power of two >= 32
    static constexpr int OUT_BYTES = (OUT == OUT_BF16) ? 2 : 1;
    static constexpr int COLS_PER_WARP = TN / (EPI_WARPS / 4);   // columns one epilogue warp covers
    // A staging row is 128 bytes (SWIZZLE_128B), or 64 (SWIZZLE_64B) where a warp's columns fill no more: e4m3
    // output from sixteen epilogue warps, 64 one-byte columns each.
    static constexpr int REGION_ROW_BYTES = (COLS_PER_WARP * OUT_BYTES < 128) ? 64 : 128;
    static constexpr int REGION_COLS = REGION_ROW_BYTES / OUT_BYTES;   // output columns in one staging row
    static constexpr int REGION_BYTES = 32 * REGION_ROW_BYTES;   // 32 rows of one warp
    static constexpr int STAGING_BYTES = EPI_WARPS * NBUF * REGION_BYTES;
    static constexpr int REGIONS_PER_TILE = COLS_PER_WARP / REGION_COLS;
    static constexpr int CHUNKS_PER_REGION = REGION_COLS / 32;   // 32-column tcgen05.ld chunks per region
    static constexpr int BAR_BYTES = 512;                        // pipeline barriers + two per staging box
    // fp32 bias of the current tile: one copy per epilogue warp in shared memory (broadcast reads) where that fits;
    // a configuration that needs every byte for the operand ring keeps it in registers instead (lane l holds the
    // bias of column l of each 32-column chunk) and broadcasts by warp shuffle.
    static constexpr bool BIAS_IN_SMEM = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + EPI_WARPS * COLS_PER_WARP * 4 + 512 <= 232448;
    static constexpr int BIAS_BYTES = BIAS_IN_SMEM ? EPI_WARPS * COLS_PER_WARP * 4 : 0;
    static constexpr int THREADS = (4 + EPI_WARPS) * 32;         // A producer, MMA, epilogue warps, side-data loader, B producer
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BIAS_BYTES + BAR_BYTES;
    static_assert(STAGE_BYTES % 1024 == 0, "every operand tile must start on a swizzle-atom boundary");
    static_assert(COLS_PER_WARP % REGION_COLS == 0, "a warp stores whole staging regions");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may use");
};

struct WaitCtx {
    volatile uint32_t* abort_flag;  // shared memory, one per CTA
    uint32_t peer_abort;            // shared::cluster address of the other CTA's flag in a CTA pair, else 0
    uint32_t* status;
    unsigned long long budget_ns;
    uint32_t tile;
};

// Polls `bar` until the phase with parity `parity` has completed.  Returns false if the CTA
// is aborting or the budget ran out (in which case it records `code` and raises the flag).
// SPIN: poll without parking the thread (the two single-thread roles on the critical path, whose wake-up
// latency is paid by the whole CTA pair); otherwise each poll may park the thread until the phase completes.
template <bool SPIN = false>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t code,
                                         uint32_t which) {
    if (SPIN ? (mbar_test_wait(bar, parity) != 0u) : mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (SPIN ? (mbar_test_wait(bar, parity) != 0u) : mbar_try_wait(bar, parity)) return true;
        if ((spins & (SPIN ? 255u : 15u)) == 0) {   // each parked poll may have lasted up to 20 us
            if (*w.abort_flag) return false;
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > w.budget_ns) {
                *w.abort_flag = 1u;
                // the other CTA of a pair would otherwise sit out its own full budget on barriers only this CTA feeds
                if (w.peer_abort) asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(w.peer_abort), "r"(1u) : "memory");
                if (atomicCAS(w.status, 0u, code) == 0u) {
                    w.status[1] = which;
                    w.status[2] = w.tile;
                    w.status[3] = blockIdx.x;
                }
                return false;
            }
        }
    }
}

// tanh-form GELU of the reference (fc1_gelu.cu:16-19) written without the 1 + tanh
// cancellation: 0.5 x (1 + tanh u) == x * sigmoid(2u) == x / (1 + exp(-2u)), with
// u = sqrt(2/pi) (x + 0.044715 x^3).  Two SFU operations (ex2, rcp) per element; everything else
// runs two elements per instruction on packed fp32 pairs.
__device__ __forceinline__ uint64_t gelu_tanh_x2(uint64_t x) {
    constexpr float K0 = -2.0f * 0.7978845608f * 1.4426950408889634f;   // -2 sqrt(2/pi) log2(e)
    constexpr float K1 = K0 * 0.044715f;
    const uint64_t x2 = mul_f32x2(x, x);
    const uint64_t t = mul_f32x2(x, fma_f32x2(x2, pack_f32x2(K1, K1), pack_f32x2(K0, K0)));   // -2 u log2(e)
    float t0, t1;
    unpack_f32x2(t, t0, t1);
    const uint64_t d = add_f32x2(pack_f32x2(ex2_approx(t0), ex2_approx(t1)), pack_f32x2(1.0f, 1.0f));
    float d0, d1;
    unpack_f32x2(d, d0, d1);
    return mul_f32x2(x, pack_f32x2(rcp_approx(d0), rcp_approx(d1)));    // x / inf == 0
}

// The same GELU through the hardware tanh (tanh.approx.f32: one SFU operation per element instead of two, relative
// error about 2^-11, so |error| <= ~2.5e-4 |x|): 0.5 x (1 + tanh u) = h + h tanh u with h = x / 2.  Opt-in
// (SL8_FLAG_GELU_HW_TANH); inside the 1e-2 relative tolerance of bf16 outputs except where the result itself is within
// ~1e-3 of zero, but not bit-comparable to the exact form.
__device__ __forceinline__ uint64_t gelu_hw_tanh_x2(uint64_t x) {
    constexpr float C0 = 0.7978845608f, C1 = 0.7978845608f * 0.044715f;
    const uint64_t x2 = mul_f32x2(x, x);
    const uint64_t u = mul_f32x2(x, fma_f32x2(x2, pack_f32x2(C1, C1), pack_f32x2(C0, C0)));
    float u0, u1;
    unpack_f32x2(u, u0, u1);
    const uint64_t h = mul_f32x2(x, pack_f32x2(0.5f, 0.5f));
    return fma_f32x2(h, pack_f32x2(tanh_approx(u0), tanh_approx(u1)), h);
}

__device__ __forceinline__ void unpack8_bf16(const uint4& q, float (&f)[8]) {
    f[0] = bf16_lo_f32(q.x); f[1] = bf16_hi_f32(q.x);
    f[2] = bf16_lo_f32(q.y); f[3] = bf16_hi_f32(q.y);
    f[4] = bf16_lo_f32(q.z); f[5] = bf16_hi_f32(q.z);
    f[6] = bf16_lo_f32(q.w); f[7] = bf16_hi_f32(q.w);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Per-warp epilogue constants.
struct EpiCtx {
    float scale;      // scale_a * scale_b
    float inv_out;    // 1 / out_scale
    uint32_t row_off; // lane * row bytes: byte offset of this lane's row inside a staging region
    uint32_t swz;     // XOR applied to the 16-byte piece index: lane & 7 (SWIZZLE_128B) or (lane >> 1) & 3 (SWIZZLE_64B)
    unsigned flags;
};

// Transforms 16 accumulator columns (v[16*H .. 16*H+15]) of this lane's row and writes them to the
// staging region at `region` (shared address), 16-byte pieces `piece0`.. of the lane's 128-byte row.
// bias16: the 16 fp32 bias values of these columns in shared memory (FC1 / FC2).  With side data
// (patch-embed table, FC2 residual) the 16 bf16 side values already sit in the staging region at the
// very place the result goes; they are read, combined and overwritten.
// Four consecutive bias values of the half-chunk: from the warp's shared copy, or (BSM false) from the chunk's
// bias register of lanes first .. first + 3.  Every lane of the warp must call it.
template <bool BSM>
__device__ __forceinline__ float4 bias_quad(const float* bias16, float breg, int first, int i) {
    if constexpr (BSM) {
        return *reinterpret_cast<const float4*>(bias16 + 4 * i);
    } else {
        float4 b;
        b.x = __shfl_sync(0xffffffffu, breg, first + 4 * i + 0);
        b.y = __shfl_sync(0xffffffffu, breg, first + 4 * i + 1);
        b.z = __shfl_sync(0xffffffffu, breg, first + 4 * i + 2);
        b.w = __shfl_sync(0xffffffffu, breg, first + 4 * i + 3);
        return b;
    }
}

template <int OP, int OUT, int H, bool BSM>
__device__ __forceinline__ void epilogue_16(const float (&v)[32], const EpiCtx& e, const float* bias16, float breg,
                                            uint32_t region, int piece0) {
    float x[16];
    uint32_t w[8];  // bf16: 8 words (16 values); e4m3: 4 words used
    const uint32_t a0 = region + e.row_off + (((piece0 + 0) ^ e.swz) << 4);
    const uint32_t a1 = region + e.row_off + (((piece0 + 1) ^ e.swz) << 4);

    if constexpr (OP == OP_PE) {
        const uint4 s0 = lds128(a0), s1 = lds128(a1);
#pragma unroll
        for (int i = 0; i < 16; i++) x[i] = v[16 * H + i] * e.scale;
        const uint32_t tw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        if (e.flags & FLAG_PE_F32_ADD) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                w[i] = pack_bf16x2(x[2 * i] + bf16_lo_f32(tw[i]), x[2 * i + 1] + bf16_hi_f32(tw[i]));
        } else {
            // The reference's order: round the accumulator to bf16, then add in bf16 (patch_embed.cu:51-58).
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = add_bf16x2(pack_bf16x2(x[2 * i], x[2 * i + 1]), tw[i]);
        }
    } else if constexpr (OP == OP_FC1) {
        // acc * scale + bias, GELU and the output scaling on packed fp32 pairs; the bias comes from shared
        // memory, the same address in every lane (a broadcast read).
        const uint64_t scale2 = pack_f32x2(e.scale, e.scale);
        const uint64_t inv2 = pack_f32x2(e.inv_out, e.inv_out);
        uint64_t g[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 b = bias_quad<BSM>(bias16, breg, 16 * H, i);
            g[2 * i + 0] = fma_f32x2(pack_f32x2(v[16 * H + 4 * i + 0], v[16 * H + 4 * i + 1]), scale2, pack_f32x2(b.x, b.y));
            g[2 * i + 1] = fma_f32x2(pack_f32x2(v[16 * H + 4 * i + 2], v[16 * H + 4 * i + 3]), scale2, pack_f32x2(b.z, b.w));
        }
        if (e.flags & FLAG_GELU_HW_TANH) {                                           // warp-uniform branches
#pragma unroll
            for (int i = 0; i < 8; i++) g[i] = gelu_hw_tanh_x2(g[i]);
        } else if (!(e.flags & FLAG_NO_ACTIVATION) && !SL8_DBG(e.flags, DBG_SKIP_GELU)) {
#pragma unroll
            for (int i = 0; i < 8; i++) g[i] = gelu_tanh_x2(g[i]);
        }
        if constexpr (OUT == OUT_BF16) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float lo, hi;
                unpack_f32x2(g[i], lo, hi);
                w[i] = pack_bf16x2(lo, hi);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float a, b, c, d;
                unpack_f32x2(mul_f32x2(g[2 * i + 0], inv2), a, b);
                unpack_f32x2(mul_f32x2(g[2 * i + 1], inv2), c, d);
                w[i] = static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
            }
        }
    } else {  // OP_FC2: (acc * scale + bias) + residual, fc2.cu:27-46
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 b = bias_quad<BSM>(bias16, breg, 16 * H, i);
            x[4 * i + 0] = fmaf(v[16 * H + 4 * i + 0], e.scale, b.x);
            x[4 * i + 1] = fmaf(v[16 * H + 4 * i + 1], e.scale, b.y);
            x[4 * i + 2] = fmaf(v[16 * H + 4 * i + 2], e.scale, b.z);
            x[4 * i + 3] = fmaf(v[16 * H + 4 * i + 3], e.scale, b.w);
        }
        float r[8];
        unpack8_bf16(lds128(a0), r);
#pragma unroll
        for (int i = 0; i < 8; i++) x[i] += r[i];
        unpack8_bf16(lds128(a1), r);
#pragma unroll
        for (int i = 0; i < 8; i++) x[8 + i] += r[i];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
    }
    sts128(a0, w[0], w[1], w[2], w[3]);
    if constexpr (OUT == OUT_BF16) sts128(a1, w[4], w[5], w[6], w[7]);
}

// FC1 on a whole 32-column chunk at once: sixteen independent element pairs go through the GELU's special-function
// chain (ex2, rcp) together, which keeps that pipe fed with only two epilogue warps per scheduler.  Used by the variants
// with up to eight epilogue warps (with sixteen, four warps per scheduler hide the chain and registers are scarce).
template <int OUT, bool BSM>
__device__ __forceinline__ void epilogue_32_fc1(const float (&v)[32], const EpiCtx& e, const float* bias32, float breg,
                                                uint32_t region, int piece0) {
    const uint64_t scale2 = pack_f32x2(e.scale, e.scale);
    uint64_t g[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 b = bias_quad<BSM>(bias32, breg, 0, i);
        g[2 * i + 0] = fma_f32x2(pack_f32x2(v[4 * i + 0], v[4 * i + 1]), scale2, pack_f32x2(b.x, b.y));
        g[2 * i + 1] = fma_f32x2(pack_f32x2(v[4 * i + 2], v[4 * i + 3]), scale2, pack_f32x2(b.z, b.w));
    }
    if (e.flags & FLAG_GELU_HW_TANH) {                                           // warp-uniform branches
#pragma unroll
        for (int i = 0; i < 16; i++) g[i] = gelu_hw_tanh_x2(g[i]);
    } else if (!(e.flags & FLAG_NO_ACTIVATION) && !SL8_DBG(e.flags, DBG_SKIP_GELU)) {
#pragma unroll
        for (int i = 0; i < 16; i++) g[i] = gelu_tanh_x2(g[i]);
    }
    if constexpr (OUT == OUT_BF16) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float lo, hi;
            unpack_f32x2(g[i], lo, hi);
            w[i] = pack_bf16x2(lo, hi);
        }
#pragma unroll
        for (int q = 0; q < 4; q++)
            sts128(region + e.row_off + (((piece0 + q) ^ e.swz) << 4), w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    } else {
        const uint64_t inv2 = pack_f32x2(e.inv_out, e.inv_out);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float a, b, c, d;
            unpack_f32x2(mul_f32x2(g[2 * i + 0], inv2), a, b);
            unpack_f32x2(mul_f32x2(g[2 * i + 1], inv2), c, d);
            w[i] = static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
        }
#pragma unroll
        for (int q = 0; q < 2; q++)
            sts128(region + e.row_off + (((piece0 + q) ^ e.swz) << 4), w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
}

// Bias values of columns col0 + lane + 32 i (i < NB) as fp32; zero past N or without a bias.
template <int NB>
__device__ __forceinline__ void load_bias(float (&b)[NB], const void* bias, unsigned flags, int col0, int lane, int N) {
#pragma unroll
    for (int i = 0; i < NB; i++) {
        const int col = col0 + lane + 32 * i;
        float val = 0.0f;
        if (bias != nullptr && col < N)
            val = (flags & FLAG_BIAS_F32) ? __ldg(static_cast<const float*>(bias) + col)
                                          : __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(bias) + col));
        b[i] = val;
    }
}

template <int CG, int TN, int TK, int STAGES, int EPI_WARPS, int OP, int OUT, int NBUF>
__global__ void __launch_bounds__((4 + EPI_WARPS) * 32, 1)
sl8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_bt, const __grid_constant__ CUtensorMap map_d,
                const __grid_constant__ CUtensorMap map_s, const KernelParams p) {
    using T = KernelTraits<CG, TN, TK, STAGES, EPI_WARPS, OUT, NBUF>;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_u32 = smem_u32(smem_raw);
    const uint32_t base = (raw_u32 + 1023u) & ~1023u;            // swizzle atoms are 1024-byte aligned
    uint8_t* const base_ptr = smem_raw + (base - raw_u32);

    const uint32_t staging_base = base + STAGES * T::STAGE_BYTES;
    const uint32_t bias_base = staging_base + T::STAGING_BYTES;
    const uint32_t bar_base = bias_base + T::BIAS_BYTES;
    // barrier block: full[STAGES] | empty[STAGES] | tmem_full[2] | tmem_empty[2] | tmem ptr | abort
    const uint32_t full_bar0 = bar_base;
    const uint32_t empty_bar0 = bar_base + 8 * STAGES;
    const uint32_t tfull_bar0 = bar_base + 16 * STAGES;
    const uint32_t tempty_bar0 = tfull_bar0 + 16;
    const uint32_t tmem_ptr_addr = tempty_bar0 + 16;
    uint8_t* const bar_ptr = base_ptr + (bar_base - base);
    volatile uint32_t* const tmem_ptr = reinterpret_cast<volatile uint32_t*>(bar_ptr + 16 * STAGES + 32);
    volatile uint32_t* const abort_flag = tmem_ptr + 1;
    const uint32_t side_bar0 = bar_base + 16 * STAGES + 48;     // (EPI_WARPS / 4) * NBUF barriers: side data landed
    const uint32_t side_free0 = side_bar0 + 8 * (EPI_WARPS / 4) * NBUF;   // ... and: staging box reusable
    static_assert(16 * STAGES + 48 + 16 * (EPI_WARPS / 4) * NBUF <= T::BAR_BYTES, "barrier block too small");

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    // Rank inside the CTA pair.  Clusters are (2,1,1) on a one-dimensional grid, so the rank is the parity of
    // blockIdx.x; taking it from there (not from %cluster_ctarank) lets the compiler see it as warp-uniform.
    const uint32_t cta_rank = (CG == 2) ? (blockIdx.x & 1u) : 0u;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;

    WaitCtx wc;
    wc.abort_flag = abort_flag;
    wc.status = p.status;
    wc.budget_ns = static_cast<unsigned long long>(p.wait_budget_us) * 1000ull;
    wc.peer_abort = (CG == 2) ? map_to_cta(smem_u32(const_cast<uint32_t*>(abort_flag)), cta_rank ^ 1u) : 0u;
    wc.tile = 0;

    // ---------------------------------------------------------------- set-up
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        prefetch_tensormap(&map_bt);
        prefetch_tensormap(&map_d);
        if constexpr (OP != OP_FC1) prefetch_tensormap(&map_s);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < STAGES; s++) {
                mbar_init(full_bar0 + 8 * s, 1);    // one arrive.expect_tx (the leader's, for the whole pair)
                mbar_init(empty_bar0 + 8 * s, 1);   // one tcgen05.commit
            }
            for (int b = 0; b < 2; b++) {
                mbar_init(tfull_bar0 + 8 * b, 1);                  // one tcgen05.commit
                mbar_init(tempty_bar0 + 8 * b, EPI_WARPS * CG);    // one arrival per epilogue warp of the pair
            }
            for (int b = 0; b < (EPI_WARPS / 4) * NBUF; b++) {
                mbar_init(side_bar0 + 8 * b, 1);     // one arrive (+ bytes) per fill of a group's box
                mbar_init(side_free0 + 8 * b, 4);    // released by the group's four warps
            }
            fence_mbar_init();
        }
        __syncwarp();
        tmem_alloc<CG>(tmem_ptr_addr, T::TMEM_COLS);
        tmem_relinquish<CG>();
    }
    tc_fence_before();
    if constexpr (CG == 2) {
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    // ---------------------------------------------------------------- roles
    if (warp == 0 || warp == 3 + EPI_WARPS) {
        // ===== TMA producers: warp 0 brings A, the last warp brings B =====
        // Both wait for the stage to be free and then issue their own copies.  Only the A producer arrives on
        // the stage's full barrier (in a CTA pair: only the leader's), announcing the bytes of everything that
        // will land on it; the other copies just count down.  The transaction count may run negative until
        // that arrive lands, and the phase cannot complete before it.  A B copy can never be a whole phase
        // ahead of the arrive it belongs to: the stage is only handed back (empty barrier) after the MMAs have
        // read it, i.e. after the previous phase of the full barrier completed, arrive included.
        if (lane == 0) {
            const bool is_a = (warp == 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const bool prof_total = p.prof != nullptr && is_a;
            const bool prof = prof_total && !(p.flags & (FLAG_COARSE_TRACE | DBG_COARSE_TRACE));
            const uint32_t full_bar_leader = (CG == 2) ? map_to_cta(full_bar0, 0) : full_bar0;
            long long t_wait = 0;
            const long long t_begin = clock64();
            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                const int tm = tile / p.tiles_n;
                const int tn = tile - tm * p.tiles_n;
                const int m0 = tm * (T::TILE_M_CTA * CG) + static_cast<int>(cta_rank) * T::TILE_M_CTA;
                // The last N tile may be narrower: each CTA of a pair then holds tail_cols / CG rows of B,
                // brought by a tensor map whose box is that tall (map_bt), and the MMAs are issued with N = tail_cols.
                const bool tail = (tn == p.tiles_n - 1) && (p.tail_cols != TN);
                const int b_rows = tail ? p.tail_cols / CG : T::B_ROWS;
                const int nb = tn * TN + static_cast<int>(cta_rank) * b_rows;
                // (measurement builds: DBG_SKIP_A / DBG_SKIP_B leave one operand's copies out; the MMAs then read stale shared memory)
                const uint32_t stage_tx = static_cast<uint32_t>((SL8_DBG(p.flags, DBG_SKIP_A) ? 0 : T::A_BYTES) +
                                                                (SL8_DBG(p.flags, DBG_SKIP_B) ? 0 : T::KATOMS * b_rows * 128));
                const bool skip_mine = is_a ? SL8_DBG(p.flags, DBG_SKIP_A) : SL8_DBG(p.flags, DBG_SKIP_B);
                const CUtensorMap* const bmap = tail ? &map_bt : &map_b;
                const int drop_kb = (!is_a && (p.flags & FLAG_TEST_DROP_B) && tile == cluster_id) ? 1 : -1;   // evaluated once per tile
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    const long long t0 = prof ? clock64() : 0;
                    ok = wait_bar<SL8_SPIN_CRITICAL>(empty_bar0 + 8 * stage, phase ^ 1u, wc, ST_PRODUCER_EMPTY_WAIT, stage);
                    if (prof) t_wait += clock64() - t0;
                    if (!ok) break;
                    const uint32_t a_dst = base + stage * T::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + T::A_BYTES;
                    if (SL8_DBG(p.flags, DBG_SKIP_LOAD)) {   // measurement aid: MMAs run on whatever shared memory holds
                        if (cta_rank == 0 && is_a) mbar_arrive(full_bar0 + 8 * stage);
                    } else if constexpr (CG == 2) {
                        const uint32_t bar = full_bar_leader + 8 * stage;
                        if (is_a) {
                            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar0 + 8 * stage, 2 * stage_tx);
                            if (!skip_mine) {
#pragma unroll
                                for (int a = 0; a < T::KATOMS; a++)
                                    tma_load_2d_pair(a_dst + a * T::A_ATOM_BYTES, &map_a, kb * T::TILE_K + 128 * a, m0, bar);
                            }
                        } else if (!skip_mine && kb != drop_kb) {
#pragma unroll
                            for (int a = 0; a < T::KATOMS; a++)
                                tma_load_2d_pair(b_dst + a * T::B_ATOM_BYTES, bmap, kb * T::TILE_K + 128 * a, nb, bar);
                        }
                    } else {
                        const uint32_t bar = full_bar0 + 8 * stage;
                        if (is_a) {
                            mbar_arrive_expect_tx(bar, stage_tx);
#pragma unroll
                            for (int a = 0; a < T::KATOMS; a++)
                                tma_load_2d(a_dst + a * T::A_ATOM_BYTES, &map_a, kb * T::TILE_K + 128 * a, m0, bar);
                        } else if (kb != drop_kb) {
#pragma unroll
                            for (int a = 0; a < T::KATOMS; a++)
                                tma_load_2d(b_dst + a * T::B_ATOM_BYTES, bmap, kb * T::TILE_K + 128 * a, nb, bar);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (prof_total) {
                long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
                slot[PROF_PRODUCER_WAIT] = t_wait;
                slot[PROF_PRODUCER_TOTAL] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===== MMA issuer (leader CTA only) =====
        // One thread.  Measured on B200: issuing one tcgen05.mma holds the thread for ~108 cycles and the MMA
        // (M 256, N 256, K 32) itself takes 128, so whatever else this thread executes per k-block (~290 cycles
        // for wait + commit + loop control when written naively) decides whether the tensor pipe idles.  Hence:
        // the poll of the NEXT stage's barrier is issued before this stage's MMAs and read after them (the
        // blocking wait runs only if that look-ahead failed), and k-blocks are taken several per loop iteration.
        if (lane == 0 && cta_rank == 0) {
            const uint32_t idesc_full = make_idesc_e4m3_f32(T::TILE_M_CTA * CG, TN);
            const uint32_t idesc_tail = make_idesc_e4m3_f32(T::TILE_M_CTA * CG, p.tail_cols);   // the last, narrower N tile
            uint32_t idesc = idesc_full;
            // Descriptors differ between stages, atoms and K steps only in the 14-bit start-address
            // field: +2 there = 32 bytes = one K = 32 step inside the 128-byte row.
            const uint64_t adesc0 = make_kmajor_sw128_desc(base);
            const uint64_t bdesc0 = make_kmajor_sw128_desc(base + T::A_BYTES);
            constexpr uint32_t STAGE_DESC = T::STAGE_BYTES >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const bool prof_any = p.prof != nullptr;
            const bool prof = prof_any && !(p.flags & (FLAG_COARSE_TRACE | DBG_COARSE_TRACE));
            long long t_full = 0, t_tmem = 0, n_tiles = 0, t_mma = 0, t_commit = 0;
            const long long t_begin = clock64();
            uint32_t ready = 0;      // look-ahead: the barrier of `stage` was already seen complete

            // All MMAs of one full k-block held in `st`; `fresh` = this k-block starts a tile (overwrite D).
            auto issue_full = [&](uint32_t d_tmem, int st, bool fresh) {
                const uint64_t adesc = adesc0 + static_cast<uint32_t>(st) * STAGE_DESC;
                const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(st) * STAGE_DESC;
#pragma unroll
                for (int j = 0; j < 4 * T::KATOMS; j++) {
                    const uint32_t o = (j >> 2) * (T::A_ATOM_BYTES >> 4) + 2 * (j & 3);
                    const uint32_t ob = (j >> 2) * (T::B_ATOM_BYTES >> 4) + 2 * (j & 3);
                    mma_f8<CG>(d_tmem, adesc + o, bdesc + ob, idesc, (j == 0 && fresh) ? 0u : 1u);
                }
            };
            auto release_stage = [&](int st) {
                if constexpr (CG == 2) mma_commit_pair(empty_bar0 + 8 * st, 0x3);
                else mma_commit(empty_bar0 + 8 * st);
            };

            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                long long t0 = prof_any ? clock64() : 0;     // once per tile: timed in the coarse mode too
                ok = wait_bar<SL8_SPIN_CRITICAL>(tempty_bar0 + 8 * acc, acc_phase ^ 1u, wc, ST_MMA_TMEM_EMPTY_WAIT, acc);
                if (prof_any) t_tmem += clock64() - t0;
                n_tiles++;
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * T::ACC_STRIDE;
                idesc = (tile % p.tiles_n == p.tiles_n - 1) ? idesc_tail : idesc_full;
                int kb = 0;
                const int k_full = p.k_blocks - 1;           // k-blocks that hold all their MMAs
                if (!prof && !SL8_DBG(p.flags, DBG_SKIP_MMA)) {
                    // One k-block: wait (only if the look-ahead failed), look ahead, MMAs, release the stage.
                    // n < 4 * KATOMS only in the K tail.
                    auto step = [&](bool fresh, int n) -> bool {
                        if (!ready) {      // the look-ahead saw the stage still filling: counted, then waited for
                            t_full++;
                            if (!wait_bar<SL8_SPIN_CRITICAL>(full_bar0 + 8 * stage, phase, wc, ST_MMA_FULL_WAIT, stage)) return false;
                        }
                        const int s1 = (stage + 1 == STAGES) ? 0 : stage + 1;
                        const uint32_t ph1 = (s1 == 0) ? (phase ^ 1u) : phase;
                        const uint32_t r1 = mbar_test_wait(full_bar0 + 8 * s1, ph1);
                        tc_fence_after();
                        if (n == 4 * T::KATOMS) {
                            issue_full(d_tmem, stage, fresh);
                        } else {
                            const uint64_t adesc = adesc0 + static_cast<uint32_t>(stage) * STAGE_DESC;
                            const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(stage) * STAGE_DESC;
#pragma unroll
                            for (int j = 0; j < 4 * T::KATOMS - 1; j++) {
                                const uint32_t o = (j >> 2) * (T::A_ATOM_BYTES >> 4) + 2 * (j & 3);
                                const uint32_t ob = (j >> 2) * (T::B_ATOM_BYTES >> 4) + 2 * (j & 3);
                                if (j < n) mma_f8<CG>(d_tmem, adesc + o, bdesc + ob, idesc, (j == 0 && fresh) ? 0u : 1u);
                            }
                        }
                        release_stage(stage);
                        stage = s1;
                        phase = ph1;
                        ready = r1;
                        return true;
                    };
                    for (; ok && kb + 2 <= k_full; kb += 2) {      // two k-blocks per loop iteration
                        ok = step(kb == 0, 4 * T::KATOMS);
                        if (ok) ok = step(false, 4 * T::KATOMS);
                    }
                    if (ok && kb < k_full) {
                        ok = step(kb == 0, 4 * T::KATOMS);
                        kb++;
                    }
                    if (ok) {
                        ok = step(kb == 0, p.last_kblock_mmas);
                        kb++;
                    }
                    if (!ok) break;
                }
                for (; kb < p.k_blocks; kb++) {
                    if (prof) t0 = clock64();
                    if (!ready) ok = wait_bar<SL8_SPIN_CRITICAL>(full_bar0 + 8 * stage, phase, wc, ST_MMA_FULL_WAIT, stage);
                    if (prof) t_full += clock64() - t0;
                    if (!ok) break;
                    const int s1 = (stage + 1 == STAGES) ? 0 : stage + 1;
                    const uint32_t ph1 = (s1 == 0) ? (phase ^ 1u) : phase;
                    ready = mbar_test_wait(full_bar0 + 8 * s1, ph1);
                    tc_fence_after();
                    long long t1 = prof ? clock64() : 0;
                    if (SL8_DBG(p.flags, DBG_SKIP_MMA)) {
                        // measurement aid: stages are released at once, the loads run at their own pace
                    } else if (kb < k_full) {
                        issue_full(d_tmem, stage, kb == 0);
                    } else {
                        const uint64_t adesc = adesc0 + static_cast<uint32_t>(stage) * STAGE_DESC;
                        const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(stage) * STAGE_DESC;
                        for (int j = 0; j < p.last_kblock_mmas; j++) {
                            const uint32_t o = (j >> 2) * (T::A_ATOM_BYTES >> 4) + 2 * (j & 3);
                            const uint32_t ob = (j >> 2) * (T::B_ATOM_BYTES >> 4) + 2 * (j & 3);
                            mma_f8<CG>(d_tmem, adesc + o, bdesc + ob, idesc, (kb | j) != 0 ? 1u : 0u);
                        }
                    }
                    if (prof) { const long long t2 = clock64(); t_mma += t2 - t1; t1 = t2; }
                    release_stage(stage);
                    if (prof) t_commit += clock64() - t1;
                    stage = s1;
                    phase = ph1;
                }
                if (!ok) break;
                if constexpr (CG == 2) mma_commit_pair(tfull_bar0 + 8 * acc, 0x3);
                else mma_commit(tfull_bar0 + 8 * acc);
                if (p.flags & FLAG_SINGLE_ACC) acc_phase ^= 1u;
                else { acc ^= 1; if (acc == 0) acc_phase ^= 1u; }
            }
            if (prof_any) {
                long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
                slot[PROF_MMA_WAIT_FULL] = t_full;
                slot[PROF_MMA_WAIT_TMEM] = t_tmem;
                slot[PROF_MMA_TOTAL] = clock64() - t_begin;
                slot[PROF_TILES] = n_tiles;
                slot[PROF_MMA_ISSUE] = t_mma;
                slot[PROF_MMA_COMMIT] = t_commit;
            }
        }
        __syncwarp();
    } else if (warp < 2 + EPI_WARPS) {
        // ===== epilogue =====
        const int ew = warp - 2;
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int col_part = ew >> 2;              // 0, or 0/1 with eight epilogue warps
        const int col_begin = col_part * T::COLS_PER_WARP;
        constexpr int RPT = T::REGIONS_PER_TILE;
        constexpr bool HAS_BIAS = (OP != OP_PE);
        constexpr bool HAS_SIDE = (OP != OP_FC1);
        static_assert(!HAS_SIDE || NBUF >= 2, "side data needs a buffer to land in while another is stored");

        EpiCtx e;
        e.scale = (p.scale_a ? __ldg(p.scale_a) : 1.0f) * (p.scale_b ? __ldg(p.scale_b) : 1.0f);
        e.inv_out = __frcp_rn(p.out_scale ? __ldg(p.out_scale) : 1.0f);   // IEEE 1/x, as the CPU oracle computes it
        e.flags = p.flags;
        e.swz = (T::REGION_ROW_BYTES == 128) ? (lane & 7) : ((lane >> 1) & 3);
        e.row_off = lane * T::REGION_ROW_BYTES;
        // Staging is organised per column group (the four quadrant warps that cover the same columns):
        // NBUF boxes of 128 rows x 128 bytes, of which this warp owns rows 32 * quad .. 32 * quad + 31.
        const uint32_t my_staging = staging_base + col_part * NBUF * 4 * T::REGION_BYTES + quad * T::REGION_BYTES;
        const long long warp_row_in_tile = static_cast<long long>(cta_rank) * T::TILE_M_CTA + quad * 32;

        const uint32_t my_side_bar = side_bar0 + 8 * col_part * NBUF;      // side data of the group's box b landed
        const uint32_t my_side_free = side_free0 + 8 * col_part * NBUF;    // the group's box b may be refilled

        constexpr int NB = T::COLS_PER_WARP / 32;  // bias values each lane stages per tile
        float* const bias_w = reinterpret_cast<float*>(base_ptr + (bias_base - base)) + ew * T::COLS_PER_WARP;
        constexpr bool BSM = T::BIAS_IN_SMEM;
        float bnext[NB], bcur[NB];
#pragma unroll
        for (int i = 0; i < NB; i++) bcur[i] = bnext[i] = 0.0f;
        if constexpr (HAS_BIAS) {
            if (cluster_id < p.num_tiles) {
                const int tn0 = cluster_id % p.tiles_n;
                load_bias<NB>(bnext, p.bias, p.flags, tn0 * TN + col_begin, lane, p.N);
#pragma unroll
                for (int i = 0; i < NB; i++) {
                    if constexpr (BSM) bias_w[lane + 32 * i] = bnext[i];
                    else bcur[i] = bnext[i];
                }
                __syncwarp();
            }
        }
        bool ok = true;
        uint32_t seq = 0;                          // regions processed so far by this warp
        int acc = 0;
        uint32_t acc_phase = 0;
        const bool prof_total = p.prof != nullptr && ew == 0;
        const bool prof = prof_total && !(p.flags & (FLAG_COARSE_TRACE | DBG_COARSE_TRACE));   // inner timers cost ~35 cycles each
        long long t_acc = 0, t_store = 0, t_ld = 0, t_math = 0, t_issue = 0, t_refill = 0;
        const long long t_begin = clock64();
        for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
            wc.tile = tile;
            const int tm = tile / p.tiles_n;
            const int tn = tile - tm * p.tiles_n;
            const long long m_warp = static_cast<long long>(tm) * (T::TILE_M_CTA * CG) + warp_row_in_tile;
            const int n0 = tn * TN;

            // The next tile's bias travels to registers while this tile is processed.
            const int next_tile = tile + num_clusters;
            const bool has_next = next_tile < p.num_tiles;
            if constexpr (HAS_BIAS) {
                if (has_next) load_bias<NB>(bnext, p.bias, p.flags, (next_tile % p.tiles_n) * TN + col_begin, lane, p.N);
            }

            // One lane polls; the others then confirm with a single try_wait of their own.
            long long t0 = prof_total ? clock64() : 0;       // once per tile: timed in the coarse mode too
            if (lane == 0) ok = wait_bar(tfull_bar0 + 8 * acc, acc_phase, wc, ST_EPI_TMEM_FULL_WAIT, acc);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok && lane != 0) ok = wait_bar(tfull_bar0 + 8 * acc, acc_phase, wc, ST_EPI_TMEM_FULL_WAIT, acc);
            ok = __all_sync(0xffffffffu, ok);
            if (prof_total) t_acc += clock64() - t0;
            if (!ok) break;
            tc_fence_after();

            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * T::ACC_STRIDE;
            const bool warp_rows_ok = m_warp < p.M;      // warp-uniform: any row of this warp inside M
            bool released = false;

#pragma unroll 1
            for (int r = 0; r < RPT; r++, seq++) {
                const int c0 = col_begin + r * T::REGION_COLS;       // first column of the region inside the tile
                const int col0 = n0 + c0;
                const uint32_t region = my_staging + (seq % NBUF) * 4 * T::REGION_BYTES;
                if (prof) t0 = clock64();
                if constexpr (HAS_SIDE) {
                    // this region's side values have landed: one lane polls, the others confirm
                    const uint32_t sbar = my_side_bar + 8 * (seq % NBUF);
                    const uint32_t spar = (seq / NBUF) & 1u;
                    if (lane == 0) ok = wait_bar(sbar, spar, wc, ST_EPI_SIDE_WAIT, seq % NBUF);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && lane != 0) ok = wait_bar(sbar, spar, wc, ST_EPI_SIDE_WAIT, seq % NBUF);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                } else {
                    if (lane == 0) tma_store_wait_read<NBUF - 1>();   // the buffer is no longer read by an older store
                    __syncwarp();
                }
                if (prof) t_store += clock64() - t0;

                const bool live = col0 < p.N && !SL8_DBG(p.flags, DBG_SKIP_EPILOGUE);   // warp-uniform
                if (live) {
#pragma unroll
                    for (int ch = 0; ch < T::CHUNKS_PER_REGION; ch++) {
                        const int c = c0 + 32 * ch;
                        if (n0 + c < p.N) {
                            float v[32];
                            if (SL8_DBG(p.flags, DBG_SKIP_TMEM_LD)) {   // measurement aid: the epilogue works on constants
#pragma unroll
                                for (int i = 0; i < 32; i++) v[i] = 1.0f;
                            } else {
                                tmem_ld_32x32(t_row + c, v);
                            }
                            if (prof) t0 = clock64();
                            if (!SL8_DBG(p.flags, DBG_SKIP_TMEM_LD)) tmem_ld_wait();
                            if (prof) t_ld += clock64() - t0;
                            if (r == RPT - 1 && ch == T::CHUNKS_PER_REGION - 1) {
                                // Last read of this accumulator: hand the TMEM buffer back before the math.
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) {
                                    if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(tempty_bar0 + 8 * acc, 0));
                                    else mbar_arrive(tempty_bar0 + 8 * acc);
                                }
                                released = true;
                            }
                            if (prof) t0 = clock64();
                            const int piece0 = ch * 2 * T::OUT_BYTES;            // 32 columns = 2 (e4m3) or 4 (bf16) pieces
                            const float* bias32 = bias_w + (c - col_begin);
                            float breg = bcur[0];                       // this chunk's bias, one column per lane
                            if constexpr (!BSM) {
#pragma unroll
                                for (int i = 1; i < NB; i++)
                                    if (i == r * T::CHUNKS_PER_REGION + ch) breg = bcur[i];
                            }
                            if (!SL8_DBG(p.flags, DBG_SKIP_MATH)) {
                                if constexpr (OP == OP_FC1 && EPI_WARPS <= 8) {
                                    // (columns past N are computed on whatever the accumulator holds and clipped by the TMA store)
                                    epilogue_32_fc1<OUT, BSM>(v, e, bias32, breg, region, piece0);
                                } else {
                                    epilogue_16<OP, OUT, 0, BSM>(v, e, bias32, breg, region, piece0);
                                    if (n0 + c + 16 < p.N) epilogue_16<OP, OUT, 1, BSM>(v, e, bias32 + 16, breg, region, piece0 + T::OUT_BYTES);
                                }
                            }
                            if (prof) t_math += clock64() - t0;
                        }
                    }
                    if (prof) t0 = clock64();
                    if (!SL8_DBG(p.flags, DBG_SKIP_STORE)) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && warp_rows_ok) tma_store_2d(&map_d, region, col0, static_cast<int>(m_warp));
                    }
                    if (prof) t_issue += clock64() - t0;
                }
                if (lane == 0) tma_store_commit();       // one bulk group per region, possibly empty
                if constexpr (HAS_SIDE) {
                    // Once the PREVIOUS region's store has read its buffer, hand that buffer back to the
                    // side-data loader (this region's store may still be reading its own).
                    if (prof) t0 = clock64();
                    if (lane == 0) {
                        tma_store_wait_read<1>();
                        if (seq > 0) mbar_arrive(my_side_free + 8 * ((seq - 1) % NBUF));
                    }
                    if (prof) t_refill += clock64() - t0;
                }
            }

            if (!ok) break;
            if (!released) {                             // tile whose last region lies past N
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(tempty_bar0 + 8 * acc, 0));
                    else mbar_arrive(tempty_bar0 + 8 * acc);
                }
            }
            if (p.flags & FLAG_SINGLE_ACC) acc_phase ^= 1u;
            else { acc ^= 1; if (acc == 0) acc_phase ^= 1u; }

            if constexpr (HAS_BIAS) {
                if (has_next) {
                    __syncwarp();                        // every lane has finished reading this tile's bias
#pragma unroll
                    for (int i = 0; i < NB; i++) {
                        if constexpr (BSM) bias_w[lane + 32 * i] = bnext[i];
                        else bcur[i] = bnext[i];
                    }
                    __syncwarp();
                }
            }
        }
        // The staging buffers must have been read before this CTA's shared memory is given back; the writes themselves
        // are complete for whoever is ordered after the kernel, as every write of a kernel is.
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        if (prof_total && lane == 0) {
            long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
            slot[PROF_EPI_WAIT_ACC] = t_acc;
            slot[PROF_EPI_WAIT_STORE] = t_store;
            slot[PROF_EPI_WAIT_LD] = t_ld;
            slot[PROF_EPI_MATH] = t_math;
            slot[PROF_EPI_STORE_ISSUE] = t_issue;
            slot[PROF_EPI_REFILL] = t_refill;
            slot[PROF_EPI_TOTAL] = clock64() - t_begin;
        }
    } else {
        // ===== side-data loader =====
        // Region number s of a column group (RPT per tile, tiles in the order this cluster visits them)
        // -> 128 rows x 128 bytes of the table / residual (the rows of this CTA's tile, 64 bf16 columns)
        // into the group's staging box s % NBUF, in the swizzled layout the TMA stores of the result
        // expect; completion on the box's "landed" barrier.  One TMA load.  A positional table that holds
        // at least period + 127 rows (rows past the period repeating it) never needs anything else; with
        // an unpadded table the boxes that wrap around its end are copied row by row by the whole warp.
        if constexpr (OP != OP_FC1) {
            constexpr int RPT = T::REGIONS_PER_TILE;
            constexpr int GROUPS = EPI_WARPS / 4;
            constexpr uint32_t BOX_BYTES = 4 * T::REGION_BYTES;
            const bool skip_side = SL8_DBG(p.flags, DBG_SKIP_SIDE);
            int my_tiles = 0;
            if (cluster_id < p.num_tiles) my_tiles = (p.num_tiles - cluster_id + num_clusters - 1) / num_clusters;
            const uint32_t total = static_cast<uint32_t>(my_tiles) * RPT;
            bool ok = true;
            for (uint32_t s = 0; ok && s < total; s++) {
                const int tile = cluster_id + static_cast<int>(s / RPT) * num_clusters;
                const int tm = tile / p.tiles_n;
                const int tn = tile - tm * p.tiles_n;
                const long long m_cta = static_cast<long long>(tm) * (T::TILE_M_CTA * CG) + cta_rank * T::TILE_M_CTA;
                wc.tile = tile;
#pragma unroll 1
                for (int g = 0; g < GROUPS; g++) {
                    const uint32_t bsel = s % NBUF;
                    const uint32_t landed = side_bar0 + 8 * (g * NBUF + bsel);
                    const uint32_t freed = side_free0 + 8 * (g * NBUF + bsel);
                    const uint32_t buf = staging_base + (g * NBUF + bsel) * BOX_BYTES;
                    // the box's previous occupant (region s - NBUF) has been stored by all four warps
                    if (lane == 0) ok = wait_bar(freed, ((s / NBUF) & 1u) ^ 1u, wc, ST_SIDE_LOADER_WAIT, g);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    const int col0 = tn * TN + g * T::COLS_PER_WARP + static_cast<int>(s % RPT) * T::REGION_COLS;
                    if (col0 >= p.N || skip_side) {
                        if (lane == 0) mbar_arrive(landed);
                        continue;
                    }
                    int y = static_cast<int>(m_cta);
                    bool wraps = false;
                    if constexpr (OP == OP_PE) {
                        y = static_cast<int>((static_cast<uint32_t>(m_cta) + static_cast<uint32_t>(p.row_phase)) % static_cast<uint32_t>(p.period));
                        wraps = y + T::TILE_M_CTA > p.table_rows;   // only a table without periodic padding wraps
                    }
                    if (!wraps) {
                        if (lane == 0) {
                            mbar_arrive_expect_tx(landed, BOX_BYTES);
                            tma_load_2d(buf, &map_s, col0, y, landed);
                        }
                    } else {
                        const int piece = lane & 7;                 // 16-byte piece (8 bf16 columns) of the 128-byte row
                        const int col = col0 + piece * 8;
                        int t = y + (lane >> 3);
                        while (t >= p.period) t -= p.period;
#pragma unroll 4
                        for (int i = 0; i < 32; i++) {
                            const int r = (lane >> 3) + 4 * i;      // staging row 0..127
                            uint4 val = make_uint4(0, 0, 0, 0);
                            if (col < p.N) val = __ldg(reinterpret_cast<const uint4*>(p.side + static_cast<long long>(t) * p.ld_side + col));
                            sts128(buf + r * 128 + ((piece ^ (r & 7)) << 4), val.x, val.y, val.z, val.w);
                            t += 4;
                            while (t >= p.period) t -= p.period;
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(landed);
                    }
                }
            }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------- exit
    tc_fence_before();
    if constexpr (CG == 2) {
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
    if (*abort_flag) {
        // Something gave up: let copies and MMAs already in flight land before the shared and
        // tensor memory they target is released.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CG>(tmem_base, T::TMEM_COLS);
    }
}

}  // namespace sl8
