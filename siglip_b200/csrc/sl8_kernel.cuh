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
enum : unsigned { FLAG_BIAS_F32 = 1u, FLAG_PE_F32_ADD = 2u };

// status[0] codes: which role gave up.
enum : uint32_t {
    ST_OK = 0,
    ST_PRODUCER_EMPTY_WAIT = 1,
    ST_MMA_FULL_WAIT = 2,
    ST_MMA_TMEM_EMPTY_WAIT = 3,
    ST_EPI_TMEM_FULL_WAIT = 4
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
    static constexpr int STAGING_BYTES = TMA_STORE ? EPI_WARPS * 2 * REGION_BYTES : 0;
    static constexpr int COLS_PER_WARP = TN / (EPI_WARPS / 4);   // columns one epilogue warp covers
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    static constexpr int BAR_BYTES = 256;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES;
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
    const uint8_t* bias;           // byte pointer to bias[0] or null
    const __nv_bfloat16* side_row; // this lane's table / residual row, or null when the row is past M
    uint8_t* out_row;              // this lane's output row (direct stores), or null when past M
    uint32_t stage_row;            // shared address of this lane's 128-byte staging row (TMA stores)
    uint32_t swz;                  // (lane & 7): XOR applied to the 16-byte chunk index
    unsigned flags;
};

// Transforms 16 accumulator columns (v[16*H .. 16*H+15] = columns col .. col+15 of this
// lane's row) and stores them.  `chunk16` is the index of the first 16-byte piece inside
// the staging row when TMA stores are used.
template <int OP, int OUT, bool TMA_STORE, int H>
__device__ __forceinline__ void epilogue_16(const float (&v)[32], const EpiRow& e, int col, uint32_t region_base,
                                            int chunk16) {
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; i++) x[i] = v[16 * H + i] * e.scale;

    uint32_t w[8];  // bf16: 8 words (16 values); e4m3: 4 words used

    if constexpr (OP == OP_PE) {
        uint4 t0 = make_uint4(0, 0, 0, 0), t1 = make_uint4(0, 0, 0, 0);
        if (e.side_row != nullptr) {
            t0 = __ldg(reinterpret_cast<const uint4*>(e.side_row + col));
            t1 = __ldg(reinterpret_cast<const uint4*>(e.side_row + col + 8));
        }
        const uint32_t tw[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
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
        // bias (same address in every lane: served as a broadcast)
        if (e.bias != nullptr) {
            if (e.flags & FLAG_BIAS_F32) {
                const float4* bp = reinterpret_cast<const float4*>(e.bias + static_cast<size_t>(col) * 4);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 b = __ldg(bp + i);
                    x[4 * i + 0] += b.x; x[4 * i + 1] += b.y; x[4 * i + 2] += b.z; x[4 * i + 3] += b.w;
                }
            } else {
                const uint4* bp = reinterpret_cast<const uint4*>(e.bias + static_cast<size_t>(col) * 2);
                float b[8];
                unpack8_bf16(__ldg(bp), b);
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] += b[i];
                unpack8_bf16(__ldg(bp + 1), b);
#pragma unroll
                for (int i = 0; i < 8; i++) x[8 + i] += b[i];
            }
        }
        if constexpr (OP == OP_FC1) {
#pragma unroll
            for (int i = 0; i < 16; i++) x[i] = gelu_tanh_fast(x[i]);
        } else {  // OP_FC2: (acc + bias) + residual, fc2.cu:27-46
            if (e.side_row != nullptr) {
                float r[8];
                unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(e.side_row + col)), r);
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] += r[i];
                unpack8_bf16(__ldg(reinterpret_cast<const uint4*>(e.side_row + col + 8)), r);
#pragma unroll
                for (int i = 0; i < 8; i++) x[8 + i] += r[i];
            }
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
    const uint32_t bar_base = staging_base + T::STAGING_BYTES;
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
                mbar_init(full_bar0 + 8 * s, CG);   // one arrive.expect_tx per CTA of the pair
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
            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                const int tm = tile / p.tiles_n;
                const int tn = tile - tm * p.tiles_n;
                const int m0 = tm * (T::TILE_M_CTA * CG) + static_cast<int>(cta_rank) * T::TILE_M_CTA;
                const int nb = tn * TN + static_cast<int>(cta_rank) * T::B_ROWS;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    ok = wait_bar(empty_bar0 + 8 * stage, phase ^ 1u, wc, ST_PRODUCER_EMPTY_WAIT, stage);
                    if (!ok) break;
                    const uint32_t a_dst = base + stage * T::STAGE_BYTES;
                    const uint32_t b_dst = a_dst + T::A_BYTES;
                    if constexpr (CG == 2) {
                        const uint32_t bar = map_to_cta(full_bar0 + 8 * stage, 0);   // the leader's barrier
                        mbar_arrive_expect_tx_cluster(bar, T::STAGE_BYTES);
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
            for (int tile = cluster_id; ok && tile < p.num_tiles; tile += num_clusters) {
                wc.tile = tile;
                ok = wait_bar(tempty_bar0 + 8 * acc, acc_phase ^ 1u, wc, ST_MMA_TMEM_EMPTY_WAIT, acc);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * T::ACC_STRIDE;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    ok = wait_bar(full_bar0 + 8 * stage, phase, wc, ST_MMA_FULL_WAIT, stage);
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
        e.bias = static_cast<const uint8_t*>(p.bias);
        e.flags = p.flags;
        e.swz = lane & 7;
        e.stage_row = lane * 128;
        const uint32_t my_staging = staging_base + ew * 2 * T::REGION_BYTES;
        uint32_t region_seq = 0;                   // staging regions used so far: selects the double buffer

        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = cluster_id; tile < p.num_tiles; tile += num_clusters) {
            wc.tile = tile;
            const int tm = tile / p.tiles_n;
            const int tn = tile - tm * p.tiles_n;
            const long long m_warp = static_cast<long long>(tm) * (T::TILE_M_CTA * CG) + cta_rank * T::TILE_M_CTA + quad * 32;
            const long long row = m_warp + lane;
            const int n0 = tn * TN;

            ok = wait_bar(tfull_bar0 + 8 * acc, acc_phase, wc, ST_EPI_TMEM_FULL_WAIT, acc);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();

            const bool row_ok = row < p.M;
            e.out_row = row_ok ? static_cast<uint8_t*>(p.D) + static_cast<size_t>(row) * p.ldd * T::OUT_BYTES : nullptr;
            if constexpr (OP == OP_PE)
                e.side_row = row_ok ? p.side + ((row + p.row_phase) % p.period) * p.ld_side : nullptr;
            else if constexpr (OP == OP_FC2)
                e.side_row = row_ok ? p.side + row * p.ld_side : nullptr;
            else
                e.side_row = nullptr;

            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * T::ACC_STRIDE;
            const bool warp_rows_ok = m_warp < p.M;      // warp-uniform: any row of this warp inside M

#pragma unroll 1
            for (int c = col_begin; c < col_begin + T::COLS_PER_WARP; c += 32) {
                const int col = n0 + c;
                if (col >= p.N) break;                   // warp-uniform: rest of the tile is past N
                float v[32];
                tmem_ld_32x32(t_row + c, v);

                uint32_t region_base = 0;
                int chunk16 = 0;
                if constexpr (TMA_STORE) {
                    const int in_region = (c - col_begin) % T::REGION_COLS;
                    if (in_region == 0) {
                        // The buffer about to be written was handed to TMA two regions ago.
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                    }
                    region_base = my_staging + (region_seq & 1u) * T::REGION_BYTES;
                    chunk16 = in_region * T::OUT_BYTES / 16;
                }
                tmem_ld_wait();

                epilogue_16<OP, OUT, TMA_STORE, 0>(v, e, col, region_base, chunk16);
                if (col + 16 < p.N)
                    epilogue_16<OP, OUT, TMA_STORE, 1>(v, e, col + 16, region_base, chunk16 + 16 * T::OUT_BYTES / 16);

                if constexpr (TMA_STORE) {
                    const int in_region = (c - col_begin) % T::REGION_COLS;
                    const bool region_done = (in_region + 32 == T::REGION_COLS) || (col + 32 >= p.N);
                    if (region_done) {
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
        }
        if constexpr (TMA_STORE) {
            if (lane == 0) tma_store_wait_all<0>();
            __syncwarp();
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
