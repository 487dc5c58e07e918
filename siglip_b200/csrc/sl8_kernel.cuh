// sl8_kernel.cuh -- the persistent, warp-specialised FP8 GEMM kernel with fused epilogues.
//
// One kernel template covers the three layers (patch-embed + periodic table add,
// FC1 + bias + GELU, FC2 + bias + residual) and every tile configuration.  It is the
// counterpart of the reference's persistent_gemm<EpilogueOp> (kernel_body.cuh:448-815) and
// epilogue_store (kernel_body.cuh:47-442), rebuilt around run-time M/N/K:
//
//   warp 0        TMA producer: streams A[128 x 128B] and B[TN/CG x 128B] k-blocks into a
//                 ring of STAGES shared-memory stages (SWIZZLE_128B), one mbarrier pair
//                 (full / empty) per stage.
//   warp 1        allocates tensor memory; one thread of the leader CTA issues
//                 tcgen05.mma kind::f8f6f4 (E4M3 x E4M3 -> FP32 in TMEM), four K=32 steps per
//                 k-block (fewer in the K tail), and commits to the stage's empty barrier and,
//                 after the last k-block, to the accumulator's full barrier.
//   warps 2..     epilogue: tcgen05.ld of the finished accumulator (two accumulators in TMEM,
//                 so the MMA of tile i+1 overlaps the epilogue of tile i), dequantisation
//                 scale, fused bias / GELU / residual / table add, conversion to bf16 or
//                 e4m3, and either direct 16-byte global stores or swizzled shared staging
//                 followed by TMA tensor stores.
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

namespace sl8 {

enum : int { OP_PE = 0, OP_FC1 = 1, OP_FC2 = 2 };
enum : int { OUT_BF16 = 0, OUT_E4M3 = 1 };
enum : unsigned { FLAG_BIAS_F32 = 1u, FLAG_PE_F32_ADD = 2u,
                  DBG_SKIP_SIDE = 0x100u, DBG_SKIP_GELU = 0x200u, DBG_SKIP_BIAS = 0x400u, DBG_SKIP_STORE = 0x800u,
                  DBG_SKIP_LOAD = 0x1000u, DBG_SKIP_EPILOGUE = 0x2000u };

// status[0] codes: which role gave up.
enum : uint32_t {
    ST_OK = 0,
    ST_PRODUCER_EMPTY_WAIT = 1,
    ST_MMA_FULL_WAIT = 2,
    ST_MMA_TMEM_EMPTY_WAIT = 3,
    ST_EPI_TMEM_FULL_WAIT = 4
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
    PROF_SLOTS = 16
};

struct KernelParams {
    long long M;
    int N;
    int K;
    int tiles_n;
    int num_tiles;
    int k_blocks;          // ceil(K / 128)
    int last_kblock_mmas;  // K = 32 steps needed in the last k-block (1..4)
    const float* scale_a;
    const float* scale_b;
    const float* out_scale;
    const void* bias;                // bf16 [N] or fp32 [N] (FLAG_BIAS_F32); may be null
    const __nv_bfloat16* side;       // table [period, N] (patch-embed) or residual [M, N] (FC2)
    long long ld_side;               // elements
    int period;
    int row_phase;
    void* D;
    long long ldd;                   // elements of the output type
    unsigned flags;
    unsigned wait_budget_ms;
    uint32_t* status;                // 4 words: code, barrier/stage, tile, block
    long long* prof;                 // optional: PROF_SLOTS clock64 totals per CTA (null = tracing off)
};

template <int CG, int TN, int STAGES, int EPI_WARPS, int OUT, bool TMA_STORE>
struct KernelTraits {
    static_assert(CG == 1 || CG == 2, "one CTA or a CTA pair per tile");
    static_assert(TN == 128 || TN == 192 || TN == 256, "tile N");
    static_assert(EPI_WARPS == 4 || EPI_WARPS == 8, "one or two warps per TMEM lane quadrant");
    static constexpr int TILE_M_CTA = 128;                       // rows per CTA = TMEM lanes
    static constexpr int TILE_K = 128;                           // bytes of K per stage = swizzle span
    static constexpr int B_ROWS = TN / CG;                       // B rows this CTA loads per stage
    static constexpr int A_BYTES = TILE_M_CTA * TILE_K;          // 16 KiB
    static constexpr int B_BYTES = B_ROWS * TILE_K;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;        // also the bytes one CTA's TMA adds per stage
    static constexpr int ACC_STRIDE = (TN <= 128) ? 128 : 256;   // TMEM columns between the two accumulators
    static constexpr int TMEM_COLS = 2 * ACC_STRIDE;             // 256 or 512: a power of two >= 32
    static constexpr int OUT_BYTES = (OUT == OUT_BF16) ? 2 : 1;
    static constexpr int REGION_COLS = 128 / OUT_BYTES;          // output columns in one 128-byte staging row
    static constexpr int REGION_BYTES = 32 * 128;                // 32 rows of one warp
    // Staging buffers per epilogue warp: two (write one while TMA reads the other) with one warp
    // per scheduler; one where a second warp on the same scheduler covers the wait instead.
    static constexpr int STAGING_BUFS = (EPI_WARPS == 8) ? 1 : 2;
    static constexpr int STAGING_BYTES = TMA_STORE ? EPI_WARPS * STAGING_BUFS * REGION_BYTES : 0;
    static constexpr int COLS_PER_WARP = TN / (EPI_WARPS / 4);   // columns one epilogue warp covers
    static constexpr int BIAS_BYTES = EPI_WARPS * COLS_PER_WARP * 4;   // fp32 bias of the current tile, one copy per warp
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BIAS_BYTES + BAR_BYTES;
    static_assert(STAGE_BYTES % 1024 == 0, "every operand tile must start on a swizzle-atom boundary");
    static_assert(COLS_PER_WARP % REGION_COLS == 0 || !TMA_STORE, "a warp stores whole staging regions");
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB a CTA may use");
};

struct WaitCtx {
    volatile uint32_t* abort_flag;  // shared memory, one per CTA
    uint32_t* status;
    unsigned long long budget_ns;
    uint32_t tile;
};

// Polls `bar` until the phase with parity `parity` has completed.  Returns false if the CTA
// is aborting or the budget ran out (in which case it records `code` and raises the flag).
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const WaitCtx& w, uint32_t code,
                                         uint32_t which) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 127u) == 0) {
            if (*w.abort_flag) return false;
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > w.budget_ns) {
                *w.abort_flag = 1u;
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
// u = sqrt(2/pi) (x + 0.044715 x^3).  Two SFU operations (ex2, rcp) per element.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float k2log2e = 2.0f * 0.7978845608f * 1.4426950408889634f;
    const float x2 = x * x;
    const float t = x * fmaf(k2log2e * 0.044715f, x2, k2log2e);  // 2 u log2(e)
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-t));
    return __fdividef(x, 1.0f + e);                               // rcp.approx + mul; x / inf == 0
}

__device__ __forceinline__ void unpack8_bf16(const uint4& q, float (&f)[8]) {
    f[0] = bf16_lo_f32(q.x); f[1] = bf16_hi_f32(q.x);
    f[2] = bf16_lo_f32(q.y); f[3] = bf16_hi_f32(q.y);
    f[4] = bf16_lo_f32(q.z); f[5] = bf16_hi_f32(q.z);
    f[6] = bf16_lo_f32(q.w); f[7] = bf16_hi_f32(q.w);
}

// Everything an epilogue warp needs that does not change inside a tile.
struct EpiRow {
    float scale;                   // scale_a * scale_b
    float inv_out;                 // 1 / out_scale
    const __nv_bfloat16* side_row; // this lane's table / residual row, or null when the row is past M
    uint8_t* out_row;              // this lane's output row (direct stores), or null when past M
    uint32_t stage_row;            // byte offset of this lane's 128-byte staging row (TMA stores)
    uint32_t swz;                  // (lane & 7): XOR applied to the 16-byte chunk index
    unsigned flags;
};

// 32 bf16 side values (table or residual) of one 32-column chunk of this lane's row; columns at
// or past N are not read.
__device__ __forceinline__ void load_side32(uint4 (&s)[4], const __nv_bfloat16* side_row, int col, int N) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        if (side_row != nullptr && col + 16 * h < N) {
            s[2 * h + 0] = __ldg(reinterpret_cast<const uint4*>(side_row + col + 16 * h));
            s[2 * h + 1] = __ldg(reinterpret_cast<const uint4*>(side_row + col + 16 * h + 8));
        } else {
            s[2 * h + 0] = make_uint4(0, 0, 0, 0);
            s[2 * h + 1] = make_uint4(0, 0, 0, 0);
        }
    }
}

// Transforms 16 accumulator columns (v[16*H .. 16*H+15] = columns col .. col+15 of this lane's row)
// and stores them.  bias16 points at the 16 fp32 bias values of these columns in shared memory
// (FC1 / FC2); side holds their 16 bf16 table / residual values (patch-embed / FC2).  `chunk16`
// is the index of the first 16-byte piece inside the staging row when TMA stores are used.
template <int OP, int OUT, bool TMA_STORE, int H>
__device__ __forceinline__ void epilogue_16(const float (&v)[32], const EpiRow& e, const float* bias16,
                                            const uint4& side_lo, const uint4& side_hi, int col, uint32_t region_base,
                                            int chunk16) {
    float x[16];
    uint32_t w[8];  // bf16: 8 words (16 values); e4m3: 4 words used

    if constexpr (OP == OP_PE) {
#pragma unroll
        for (int i = 0; i < 16; i++) x[i] = v[16 * H + i] * e.scale;
        const uint32_t tw[8] = {side_lo.x, side_lo.y, side_lo.z, side_lo.w, side_hi.x, side_hi.y, side_hi.z, side_hi.w};
        if (e.flags & FLAG_PE_F32_ADD) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                w[i] = pack_bf16x2(x[2 * i] + bf16_lo_f32(tw[i]), x[2 * i + 1] + bf16_hi_f32(tw[i]));
        } else {
            // The reference's order: round the accumulator to bf16, then add in bf16 (patch_embed.cu:51-58).
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = add_bf16x2(pack_bf16x2(x[2 * i], x[2 * i + 1]), tw[i]);
        }
    } else {
        // acc * scale + bias in one FMA; the bias comes from shared memory, the same address in every
        // lane (a broadcast read).
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 b = *reinterpret_cast<const float4*>(bias16 + 4 * i);
            x[4 * i + 0] = fmaf(v[16 * H + 4 * i + 0], e.scale, b.x);
            x[4 * i + 1] = fmaf(v[16 * H + 4 * i + 1], e.scale, b.y);
            x[4 * i + 2] = fmaf(v[16 * H + 4 * i + 2], e.scale, b.z);
            x[4 * i + 3] = fmaf(v[16 * H + 4 * i + 3], e.scale, b.w);
        }
        if constexpr (OP == OP_FC1) {
            if (!(e.flags & DBG_SKIP_GELU)) {
#pragma unroll
                for (int i = 0; i < 16; i++) x[i] = gelu_tanh_fast(x[i]);
            }
        } else {  // OP_FC2: (acc + bias) + residual, fc2.cu:27-46
            float r[8];
            unpack8_bf16(side_lo, r);
#pragma unroll
            for (int i = 0; i < 8; i++) x[i] += r[i];
            unpack8_bf16(side_hi, r);
#pragma unroll
            for (int i = 0; i < 8; i++) x[8 + i] += r[i];
        }
        if constexpr (OUT == OUT_BF16) {
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = pack_bf16x2(x[2 * i], x[2 * i + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t lo = pack_e4m3x2(x[4 * i + 0] * e.inv_out, x[4 * i + 1] * e.inv_out);
                const uint32_t hi = pack_e4m3x2(x[4 * i + 2] * e.inv_out, x[4 * i + 3] * e.inv_out);
                w[i] = lo | (hi << 16);
            }
        }
    }

    constexpr int PIECES = (OUT == OUT_BF16) ? 2 : 1;  // 16-byte pieces for 16 columns
    if constexpr (TMA_STORE) {
#pragma unroll
        for (int p = 0; p < PIECES; p++) {
            const uint32_t addr = region_base + e.stage_row + (((chunk16 + p) ^ e.swz) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * p + 0]), "r"(w[4 * p + 1]),
                         "r"(w[4 * p + 2]), "r"(w[4 * p + 3])
                         : "memory");
        }
    } else {
        if (e.out_row != nullptr) {
            uint4* dst = reinterpret_cast<uint4*>(e.out_row + static_cast<size_t>(col) * ((OUT == OUT_BF16) ? 2 : 1));
#pragma unroll
            for (int p = 0; p < PIECES; p++) dst[p] = make_uint4(w[4 * p + 0], w[4 * p + 1], w[4 * p + 2], w[4 * p + 3]);
        }
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

template <int CG, int TN, int STAGES, int EPI_WARPS, int OP, int OUT, bool TMA_STORE>
__global__ void __launch_bounds__((2 + EPI_WARPS) * 32, 1)
sl8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_d, const KernelParams p) {
    using T = KernelTraits<CG, TN, STAGES, EPI_WARPS, OUT, TMA_STORE>;

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
    static_assert(16 * STAGES + 32 + 8 <= T::BAR_BYTES, "barrier block too small");

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;

    WaitCtx wc;
    wc.abort_flag = abort_flag;
    wc.status = p.status;
    wc.budget_ns = static_cast<unsigned long long>(p.wait_budget_ms) * 1000000ull;
    wc.tile = 0;

    // ---------------------------------------------------------------- set-up
    if (threadIdx.x == 0) {
        *abort_flag = 0u;
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if constexpr (TMA_STORE) prefetch_tensormap(&map_d);
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
    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const bool prof = p.prof != nullptr;
            const uint32_t full_bar_leader = (CG == 2) ? map_to_cta(full_bar0, 0) : full_bar0;
            long long t_wait = 0;
            const long long t_begin = clock64();
            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                const int tm = tile / p.tiles_n;
                const int tn = tile - tm * p.tiles_n;
                const int m0 = tm * (T::TILE_M_CTA * CG) + static_cast<int>(cta_rank) * T::TILE_M_CTA;
                const int nb = tn * TN + static_cast<int>(cta_rank) * T::B_ROWS;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    const long long t0 = prof ? clock64() : 0;
                    ok = wait_bar(empty_bar0 + 8 * stage, phase ^ 1u, wc, ST_PRODUCER_EMPTY_WAIT, stage);
                    if (prof) t_wait += clock64() - t0;
                    if (!ok) break;
                    const uint32_t a_dst = base + stage * T::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + T::A_BYTES;
                    if (p.flags & DBG_SKIP_LOAD) {   // measurement aid: MMAs run on whatever shared memory holds
                        if (cta_rank == 0) mbar_arrive(full_bar0 + 8 * stage);
                    } else if constexpr (CG == 2) {
                        // Both CTAs' copies complete on the LEADER's barrier.  Only the leader arrives on it,
                        // announcing the bytes of the whole pair; the peer's copies just count down (the
                        // transaction count may run negative until the leader's arrive lands, and the phase
                        // cannot complete before that arrive).
                        const uint32_t bar = full_bar_leader + 8 * stage;
                        if (cta_rank == 0) mbar_arrive_expect_tx(full_bar0 + 8 * stage, 2 * T::STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &map_a, kb * T::TILE_K, m0, bar);
                        tma_load_2d_pair(b_dst, &map_b, kb * T::TILE_K, nb, bar);
                    } else {
                        const uint32_t bar = full_bar0 + 8 * stage;
                        mbar_arrive_expect_tx(bar, T::STAGE_BYTES);
                        tma_load_2d(a_dst, &map_a, kb * T::TILE_K, m0, bar);
                        tma_load_2d(b_dst, &map_b, kb * T::TILE_K, nb, bar);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (prof) {
                long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
                slot[PROF_PRODUCER_WAIT] = t_wait;
                slot[PROF_PRODUCER_TOTAL] = clock64() - t_begin;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===== MMA issuer (leader CTA only) =====
        if (lane == 0 && cta_rank == 0) {
            const uint32_t idesc = make_idesc_e4m3_f32(T::TILE_M_CTA * CG, TN);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const bool prof = p.prof != nullptr;
            long long t_full = 0, t_tmem = 0, n_tiles = 0;
            const long long t_begin = clock64();
            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                long long t0 = prof ? clock64() : 0;
                ok = wait_bar(tempty_bar0 + 8 * acc, acc_phase ^ 1u, wc, ST_MMA_TMEM_EMPTY_WAIT, acc);
                if (prof) { t_tmem += clock64() - t0; n_tiles++; }
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * T::ACC_STRIDE;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    t0 = prof ? clock64() : 0;
                    ok = wait_bar(full_bar0 + 8 * stage, phase, wc, ST_MMA_FULL_WAIT, stage);
                    if (prof) t_full += clock64() - t0;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_src = base + stage * T::STAGE_BYTES;
                    const uint64_t adesc = make_kmajor_sw128_desc(a_src);
                    const uint64_t bdesc = make_kmajor_sw128_desc(a_src + T::A_BYTES);
                    const int nmma = (kb == p.k_blocks - 1) ? p.last_kblock_mmas : 4;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (j < nmma)   // +2 in the address field = 32 bytes = one K step
                            mma_f8<CG>(d_tmem, adesc + 2u * j, bdesc + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u);
                    }
                    if constexpr (CG == 2) mma_commit_pair(empty_bar0 + 8 * stage, 0x3);
                    else mma_commit(empty_bar0 + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if constexpr (CG == 2) mma_commit_pair(tfull_bar0 + 8 * acc, 0x3);
                else mma_commit(tfull_bar0 + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
            if (prof) {
                long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
                slot[PROF_MMA_WAIT_FULL] = t_full;
                slot[PROF_MMA_WAIT_TMEM] = t_tmem;
                slot[PROF_MMA_TOTAL] = clock64() - t_begin;
                slot[PROF_TILES] = n_tiles;
            }
        }
        __syncwarp();
    } else {
        // ===== epilogue =====
        const int ew = warp - 2;
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const int col_part = ew >> 2;              // 0, or 0/1 with eight epilogue warps
        const int col_begin = col_part * T::COLS_PER_WARP;

        EpiRow e;
        e.scale = (p.scale_a ? __ldg(p.scale_a) : 1.0f) * (p.scale_b ? __ldg(p.scale_b) : 1.0f);
        e.inv_out = __frcp_rn(p.out_scale ? __ldg(p.out_scale) : 1.0f);   // IEEE 1/x, as the CPU oracle computes it
        e.flags = p.flags;
        e.swz = lane & 7;
        e.stage_row = lane * 128;
        e.side_row = nullptr;
        const uint32_t my_staging = staging_base + ew * T::STAGING_BUFS * T::REGION_BYTES;
        uint32_t region_seq = 0;                   // staging regions used so far: selects the buffer

        constexpr bool HAS_BIAS = (OP != OP_PE);
        constexpr bool HAS_SIDE = (OP != OP_FC1);
        constexpr int NB = T::COLS_PER_WARP / 32;  // bias values each lane stages per tile
        float* const bias_w = reinterpret_cast<float*>(base_ptr + (bias_base - base)) + ew * T::COLS_PER_WARP;
        float bnext[NB];
        if constexpr (HAS_BIAS) {
            if (cluster_id < p.num_tiles) {
                const int tn0 = cluster_id % p.tiles_n;
                load_bias<NB>(bnext, p.bias, p.flags, tn0 * TN + col_begin, lane, p.N);
#pragma unroll
                for (int i = 0; i < NB; i++) bias_w[lane + 32 * i] = bnext[i];
                __syncwarp();
            }
        }

        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const bool prof = p.prof != nullptr && ew == 0;
        long long t_acc = 0, t_store = 0, t_ld = 0;
        const long long t_begin = clock64();
        for (int tile = cluster_id; tile < p.num_tiles; tile += num_clusters) {
            wc.tile = tile;
            const int tm = tile / p.tiles_n;
            const int tn = tile - tm * p.tiles_n;
            const long long m_warp = static_cast<long long>(tm) * (T::TILE_M_CTA * CG) + cta_rank * T::TILE_M_CTA + quad * 32;
            const long long row = m_warp + lane;
            const int n0 = tn * TN;

            // Work for the NEXT tile that can overlap this one: its bias (registers now, shared memory
            // once this tile is done) and, for FC2, an L2 prefetch of this lane's residual row segment.
            const int next_tile = tile + num_clusters;
            const bool has_next = next_tile < p.num_tiles;
            if (has_next && (HAS_BIAS || OP == OP_FC2)) {
                const int ntm = next_tile / p.tiles_n;
                const int ntn = next_tile - ntm * p.tiles_n;
                if constexpr (HAS_BIAS) load_bias<NB>(bnext, p.bias, p.flags, ntn * TN + col_begin, lane, p.N);
                if constexpr (OP == OP_FC2) {
                    const long long nrow = static_cast<long long>(ntm) * (T::TILE_M_CTA * CG) + cta_rank * T::TILE_M_CTA + quad * 32 + lane;
                    if (nrow < p.M && !(p.flags & DBG_SKIP_SIDE)) {
                        const __nv_bfloat16* r = p.side + nrow * p.ld_side + ntn * TN + col_begin;
#pragma unroll
                        for (int j = 0; j < T::COLS_PER_WARP / 64; j++)
                            if (ntn * TN + col_begin + 64 * j < p.N)
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(r + 64 * j));
                    }
                }
            }

            const bool row_ok = row < p.M;
            e.out_row = row_ok ? static_cast<uint8_t*>(p.D) + static_cast<size_t>(row) * p.ldd * T::OUT_BYTES : nullptr;
            if constexpr (OP == OP_PE)
                e.side_row = row_ok ? p.side + ((row + p.row_phase) % p.period) * p.ld_side : nullptr;
            else if constexpr (OP == OP_FC2)
                e.side_row = row_ok ? p.side + row * p.ld_side : nullptr;
            if (p.flags & DBG_SKIP_SIDE) e.side_row = nullptr;

            // Side values of the first chunk are requested before the accumulator is waited for.
            uint4 side_cur[4], side_nxt[4];
            if constexpr (HAS_SIDE) load_side32(side_cur, e.side_row, n0 + col_begin, p.N);

            long long t0 = prof ? clock64() : 0;
            ok = wait_bar(tfull_bar0 + 8 * acc, acc_phase, wc, ST_EPI_TMEM_FULL_WAIT, acc);
            ok = __all_sync(0xffffffffu, ok);
            if (prof) t_acc += clock64() - t0;
            if (!ok) break;
            tc_fence_after();

            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * T::ACC_STRIDE;
            const bool warp_rows_ok = m_warp < p.M;      // warp-uniform: any row of this warp inside M

#pragma unroll 1
            for (int c = col_begin; c < col_begin + T::COLS_PER_WARP; c += 32) {
                const int col = n0 + c;
                if (col >= p.N || (p.flags & DBG_SKIP_EPILOGUE)) break;   // warp-uniform: rest of the tile is past N
                float v[32];
                tmem_ld_32x32(t_row + c, v);
                // next chunk's side values travel while this chunk is computed
                if constexpr (HAS_SIDE) {
                    if (c + 32 < col_begin + T::COLS_PER_WARP) load_side32(side_nxt, e.side_row, col + 32, p.N);
                }

                uint32_t region_base = 0;
                int chunk16 = 0;
                if constexpr (TMA_STORE) {
                    const int in_region = (c - col_begin) % T::REGION_COLS;
                    if (in_region == 0) {
                        // The buffer about to be written must no longer be read by an earlier TMA store.
                        t0 = prof ? clock64() : 0;
                        if (lane == 0) tma_store_wait_read<T::STAGING_BUFS - 1>();
                        __syncwarp();
                        if (prof) t_store += clock64() - t0;
                    }
                    region_base = my_staging + (region_seq % T::STAGING_BUFS) * T::REGION_BYTES;
                    chunk16 = in_region * T::OUT_BYTES / 16;
                }
                t0 = prof ? clock64() : 0;
                tmem_ld_wait();
                if (prof) t_ld += clock64() - t0;

                const float* bias32 = bias_w + (c - col_begin);
                epilogue_16<OP, OUT, TMA_STORE, 0>(v, e, bias32, side_cur[0], side_cur[1], col, region_base, chunk16);
                if (col + 16 < p.N)
                    epilogue_16<OP, OUT, TMA_STORE, 1>(v, e, bias32 + 16, side_cur[2], side_cur[3], col + 16, region_base,
                                                       chunk16 + T::OUT_BYTES);
                if constexpr (HAS_SIDE) {
#pragma unroll
                    for (int i = 0; i < 4; i++) side_cur[i] = side_nxt[i];
                }

                if constexpr (TMA_STORE) {
                    const int in_region = (c - col_begin) % T::REGION_COLS;
                    const bool region_done = (in_region + 32 == T::REGION_COLS) || (col + 32 >= p.N);
                    if (region_done && !(p.flags & DBG_SKIP_STORE)) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && warp_rows_ok) {
                            tma_store_2d(&map_d, region_base, col - in_region, static_cast<int>(m_warp));
                            tma_store_commit();
                        }
                        region_seq++;
                    }
                }
            }

            // The accumulator is in registers / on its way out: hand the TMEM buffer back.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (CG == 2) mbar_arrive_cluster(map_to_cta(tempty_bar0 + 8 * acc, 0));
                else mbar_arrive(tempty_bar0 + 8 * acc);
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;

            if constexpr (HAS_BIAS) {
                if (has_next) {   // every lane has finished reading this tile's bias (the __syncwarp above)
#pragma unroll
                    for (int i = 0; i < NB; i++) bias_w[lane + 32 * i] = bnext[i];
                    __syncwarp();
                }
            }
        }
        if constexpr (TMA_STORE) {
            if (lane == 0) tma_store_wait_all<0>();
            __syncwarp();
        }
        if (prof && lane == 0) {
            long long* slot = p.prof + static_cast<size_t>(blockIdx.x) * PROF_SLOTS;
            slot[PROF_EPI_WAIT_ACC] = t_acc;
            slot[PROF_EPI_WAIT_STORE] = t_store;
            slot[PROF_EPI_WAIT_LD] = t_ld;
            slot[PROF_EPI_TOTAL] = clock64() - t_begin;
        }
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
