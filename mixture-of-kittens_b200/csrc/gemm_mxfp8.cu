// Grouped MXFP8 GEMM for the routed experts: E4M3 operands with one E8M0 scale per 32
// elements of the contraction axis, multiplied by tcgen05.mma kind::mxf8f6f4.block_scale
// with fp32 accumulation in tensor memory and bf16 output
// (reference: csrc/megakernel/grouped_gemm.cuh:183-237, the MXFP8 branches).
//
// Every MXFP8 product of the layer is "A * B^T with the contraction axis contiguous in both
// operands": the backward pass gets pre-transposed, pre-quantised weights and token-axis
// quantised activations (csrc/megakernel/backward.cuh:335-403).  So there is one operand layout
// and three ways of walking it:
//   FMODE_NT     D[rows,N] = A[rows,K] * W[g][N,K]^T (+ A2 * W2[g]^T)   down, both input gradients
//   FMODE_DUALB  D = A * Wg[g]^T, D2 = A * Wu[g]^T, one 128+128 column tile  gate and up
//   FMODE_WGRAD  D[g][M,N] = A[M, cols_g] * B[N, cols_g]^T                weight gradients
//   FMODE_GATEUP_QUANT  the products of FMODE_DUALB, kept on chip: the epilogue rounds gate and up to bf16,
//                computes hidden = SwiGLU(gate, up) and writes the MXFP8 forms the layer saves and consumes
//                (gate, up, hidden quantised along columns; hidden also along tokens) instead of bf16 gate / up
//                (the reference fuses the same quantisation into its gate/up epilogue, grouped_gemm.cuh:295-359)
//   FMODE_FWD    FMODE_GATEUP_QUANT tiles and the FMODE_NT (down) tiles of the same rows in ONE persistent launch, window
//                by window, tied by the global-memory counters described in gemm.cu (the task loop of the reference's
//                forward megakernel, csrc/megakernel/forward.cuh:146-266); the down tiles read the E4M3 hidden rows
//                and scales that the gate/up tiles of the same 256-row block have just written
//
// A CTA pair (cluster of 2, cta_group::2) computes a 256 x 256 tile; K advances 128 bytes per
// stage (4 MMAs of K = 32).  Per stage each CTA stages 16 KB of A, 16 KB of B and three
// 512-byte scale tiles (its 128 rows of A, all 256 columns of B: every CTA fetches both B scale
// tiles itself).  The MMA lane copies the scale tiles into tensor memory with tcgen05.cp
// before the stage's MMAs; the instruction descriptor's scale ids select the byte of the K block.
//
// Tensor memory: block scaling needs columns for the scales, so two 256-column accumulators do
// not fit in the 512 columns.  There is one accumulator; the epilogue drains it into registers
// as packed bf16 (about as long as one K stage), releases it, and only then writes global
// memory, so the stores still overlap the next tile's main loop.
#include <string.h>

#include "common.cuh"
#include "mxfp8_codec.cuh"

namespace mokb {
namespace {

constexpr int BN = 256, BKB = 128;                 // tile columns; K bytes (= elements) per stage
constexpr int TILE_M = 256;
constexpr int A_BYTES = 128 * BKB;                 // 16 KB per CTA
constexpr int B_BYTES = 128 * BKB;                 // 16 KB per CTA
constexpr int DATA_BYTES = A_BYTES + B_BYTES;
constexpr int SF_TILE = 512;                       // one 32 x 16-byte scale tile
constexpr int SF_BYTES = 3 * SF_TILE;              // SFA | SFB(cols 0..127) | SFB(cols 128..255)
constexpr int STAGES = 6;
constexpr int STAGE_TX = DATA_BYTES + SF_BYTES;    // bytes one CTA lands per stage
constexpr int NUM_THREADS = 320;                  // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)
constexpr int TMEM_COLS = 512;
constexpr int SF_COL0 = 256;                       // scale columns start after the accumulator
constexpr int SF_SET_COLS = 16;                    // SFA 4 + SFB 8, padded
constexpr int GROUP_M = 4;
// + one 2 KB transposition buffer per epilogue warp (32 rows x 64 bytes) for rows that are pushed to a peer
constexpr size_t SMEM_BYTES = static_cast<size_t>(STAGES) * (DATA_BYTES + SF_BYTES) + 1024 + 256 + 8 * 2048;

enum { FMODE_NT = 0, FMODE_DUALB = 1, FMODE_WGRAD = 2, FMODE_GATEUP_QUANT = 3, FMODE_FWD = 4 };
template <int MODE> constexpr bool kGateUp = MODE == FMODE_DUALB || MODE == FMODE_GATEUP_QUANT;

struct FParams {
    int rows_cap, row_begin, row_end;
    const int32_t* num_rows;
    const int32_t* group_of_block;
    const int32_t* group_offsets;
    int G, M, N, K;
    int b_rows_per_group;
    int dual;
    int a_ktiles, b_ktiles;          // scale tiles per row block of A / B (= contraction extent / 128)
    __nv_bfloat16 *D, *D2;
    int ldd;
    int wide_stores;                 // D (and D2) rows are 32-byte aligned: the epilogue stores 32 bytes per instruction
    int accumulate;                  // FMODE_WGRAD: add to the stored bf16 result instead of overwriting it
    int k_tile_origin;               // FMODE_WGRAD: the operands' first token column, in 128-token tiles, in group_offsets' row space
    // FMODE_GATEUP_QUANT outputs: E4M3 [rows, N] + packed scales for gate, up, hidden; hidden also as [N, t_rows]
    uint8_t *gate_q, *gate_sc, *up_q, *up_sc, *hid_q, *hid_sc, *hid_qt, *hid_sct;
    int t_rows;
    int has_limit;
    float limit;
    // counters (row-tiled modes; see gemm.cu) and the down projection of FMODE_FWD
    int window_rows;
    const int32_t* win_ready;
    int win_ready_target;
    int N2, K2, b3_rows_per_group, a2_ktiles, b3_ktiles;     // down: N2 columns, contraction K2 = N
    int32_t* blk_done;
    int32_t* win_done;
    int reserve_pairs;               // SM pairs a waiting launch leaves to the kernels it waits for
    // push (FMODE_NT and the down tiles of FMODE_FWD): row r goes to row push_idx[r] of rank push_rank[r]'s buffer
    int push, push_ranks, push_wide, push_limit;
    const int32_t* push_rank;
    const int32_t* push_idx;
    const float* push_values;
    int32_t* status;
    PeerPtrs push_dst, push_val;
};

struct Tile {
    int m_blk, n_blk, group, k_iters, k_tile0;
    int phase, window;               // FMODE_FWD: 0 = gate/up tile, 1 = down tile; window of the rows, from row_begin
};

template <int MODE>
struct Sched {
    int m_blocks, n_blocks, total, m_first;
    int n_gu, n_nt, win_blocks;
    __device__ Sched(const FParams& p) {
        m_first = 0;
        n_gu = n_nt = 0;
        win_blocks = 1 << 30;
        if (MODE == FMODE_WGRAD) {
            m_blocks = (p.M + TILE_M - 1) / TILE_M;
            n_blocks = (p.N + BN - 1) / BN;
            total = p.G * m_blocks * n_blocks;
            // accumulating over no token columns at all (an empty macrobatch) leaves every gradient as it is: no tiles
            if (p.accumulate && p.group_offsets[p.G] == p.group_offsets[0]) total = 0;
        } else {
            int rows = p.num_rows ? *p.num_rows : p.rows_cap;
            if (rows < 0) rows = 0;                 // the row window below never exceeds the tensors (row_end <= rows_cap)
            const int hi = min(rows, p.row_end), lo = min(p.row_begin, hi);
            m_first = lo / TILE_M;
            m_blocks = (hi - lo) / TILE_M;
            n_blocks = kGateUp<MODE> ? p.N / 128 : (p.N + BN - 1) / BN;
            total = m_blocks * n_blocks;
            if (p.window_rows > 0) win_blocks = p.window_rows / TILE_M;
            if (MODE == FMODE_FWD) {
                n_gu = p.N / 128;
                n_nt = p.N2 / BN;
                total = m_blocks * (n_gu + n_nt);
            }
        }
    }
    __device__ Tile get(const FParams& p, int t) const {
        Tile ti;
        if (MODE == FMODE_WGRAD) {
            const int per = m_blocks * n_blocks;
            ti.group = t / per;
            const int rem = t - ti.group * per;
            ti.n_blk = rem / m_blocks;
            ti.m_blk = rem - ti.n_blk * m_blocks;
            const int c0 = p.group_offsets[ti.group];
            ti.k_tile0 = c0 / BKB - p.k_tile_origin;
            ti.k_iters = (p.group_offsets[ti.group + 1] - c0) / BKB;
        } else if (MODE == FMODE_FWD) {
            const int wb = min(win_blocks, m_blocks);
            const int per_win = wb * (n_gu + n_nt);
            const int n_win = (m_blocks + wb - 1) / wb;
            const int w = min(t / per_win, n_win - 1);
            int local = t - w * per_win;
            const int blk0 = w * wb;
            const int wc = min(wb, m_blocks - blk0);
            ti.phase = local >= wc * n_gu ? 1 : 0;
            if (ti.phase) local -= wc * n_gu;
            const int nb = ti.phase ? n_nt : n_gu;
            const int per = GROUP_M * nb;
            const int sg = local / per;
            const int first = sg * GROUP_M;
            const int gsize = min(GROUP_M, wc - first);
            const int in = local - sg * per;
            ti.n_blk = in / gsize;
            ti.m_blk = m_first + blk0 + first + (in - ti.n_blk * gsize);
            ti.window = w;
            ti.group = p.group_of_block ? p.group_of_block[ti.m_blk * 2] : 0;
            ti.k_tile0 = 0;
            ti.k_iters = (ti.phase ? p.K2 : p.K) / BKB;
        } else {
            const int per = GROUP_M * n_blocks;
            const int sg = t / per;
            const int first = sg * GROUP_M;
            const int gsize = min(GROUP_M, m_blocks - first);
            const int in = t - sg * per;
            ti.n_blk = in / gsize;
            ti.m_blk = m_first + first + (in - ti.n_blk * gsize);
            ti.group = p.group_of_block ? p.group_of_block[ti.m_blk * 2] : 0;
            ti.k_tile0 = 0;
            ti.k_iters = (p.K / BKB) * (p.dual ? 2 : 1);
            ti.phase = 0;
            ti.window = (ti.m_blk - m_first) / win_blocks;
        }
        return ti;
    }
};

__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 32-byte store: one full sector per thread (the output rows are 32-byte aligned when the host sets wide_stores)
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

// 64 consecutive columns of one row (32 bf16 pairs in registers) -> two 32-element MXFP8 blocks of q [rows, N]
__device__ __forceinline__ void quantize_row_blocks(const uint32_t (&w)[32], uint8_t* q, uint8_t* sc, int64_t row, int64_t col0, int64_t N) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
        uint32_t m = 0u;
#pragma unroll
        for (int j = 0; j < 16; ++j) m = absmax2(m, w[b * 16 + j]);
        float inv;
        const uint32_t byte = scale_byte(fmaxf(bf16_lo(m), bf16_hi(m)), &inv);
        uint32_t out[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            out[j] = e4m3x4(bf16_lo(w[b * 16 + 2 * j]) * inv, bf16_hi(w[b * 16 + 2 * j]) * inv,
                            bf16_lo(w[b * 16 + 2 * j + 1]) * inv, bf16_hi(w[b * 16 + 2 * j + 1]) * inv);
        st_global_32B(q + row * N + col0 + b * 32, out);
        sc[scale_offset(row, (col0 >> 5) + b, N >> 7)] = static_cast<uint8_t>(byte);
    }
}

struct Maps {        // by-value kernel argument
    CUtensorMap A, B, A2, B2;          // E4M3 data, 128-byte swizzle, boxes of 128 x 128
    CUtensorMap SA, SB, SA2, SB2;      // scale tiles: rows of 128 u32
    CUtensorMap B3, SB3;               // FMODE_FWD: the down weights (A2 / SA2 are then the hidden rows)
};

// 128 registers per thread at most (see gemm.cu): ten warps put three on an SM quarter, and the blocks of the
// dispatch and quantise kernels that this GEMM may be waiting for have to fit beside them.
template <int MODE>
__global__ void __maxnreg__(128)
grouped_gemm_mxfp8_kernel(const __grid_constant__ Maps tm, const FParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sf_base = smem_base + STAGES * DATA_BYTES;
    const uint32_t bars = sf_base + STAGES * SF_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t tfull_bar = bars + 8u * (2 * STAGES);
    const uint32_t tempty_bar = bars + 8u * (2 * STAGES + 1);
    uint8_t* bar_gen = smem_gen + STAGES * (DATA_BYTES + SF_BYTES);
    volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * STAGES + 2));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * STAGES + 2) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();
    const int tile_id0 = static_cast<int>(blockIdx.x >> 1);
    const int tile_stride = static_cast<int>(gridDim.x >> 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        mbar_init(tempty_bar, 16);            // one arrival per epilogue warp of the pair
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm.A); tma_prefetch_desc(&tm.B); tma_prefetch_desc(&tm.SA); tma_prefetch_desc(&tm.SB);
        if (kGateUp<MODE> || p.dual) { tma_prefetch_desc(&tm.B2); tma_prefetch_desc(&tm.SB2); }
        if (p.dual) { tma_prefetch_desc(&tm.A2); tma_prefetch_desc(&tm.SA2); }
        if (MODE == FMODE_FWD) {
            tma_prefetch_desc(&tm.B2); tma_prefetch_desc(&tm.SB2);
            if (p.N2 > 0) { tma_prefetch_desc(&tm.A2); tma_prefetch_desc(&tm.SA2); tma_prefetch_desc(&tm.B3); tma_prefetch_desc(&tm.SB3); }
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_slot;

    const Sched<MODE> sched(p);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const int kh = p.K / BKB;
            int waited_window = -1;
            Tile next_ti = {};         // worked out one tile ahead: the look-up would otherwise stall short tiles
            if (tile_id0 < sched.total) next_ti = sched.get(p, tile_id0);
            for (int t = tile_id0; ok && t < sched.total; t += tile_stride) {
                const Tile ti = next_ti;
                if (t + tile_stride < sched.total) next_ti = sched.get(p, t + tile_stride);
                const int row0 = ti.m_blk * TILE_M + static_cast<int>(cta) * 128;     // this CTA's rows of A (and of D)
                if (MODE != FMODE_WGRAD) {
                    // rows that another kernel (or, for a down tile, other CTAs of this one) is still producing
                    bool fenced = false;
                    if (p.win_ready && ti.phase == 0 && ti.window > waited_window) {
                        if (!flag_wait(p.win_ready + ti.window, p.win_ready_target, abort_flag, p.status, kWaitWindowReady, ti.window)) { ok = false; break; }
                        waited_window = ti.window;
                        fenced = true;
                    }
                    if (MODE == FMODE_FWD && ti.phase == 1) {
                        if (!flag_wait(p.blk_done + (ti.m_blk - sched.m_first), sched.n_gu * 16, abort_flag, p.status, kWaitBlockDone, ti.m_blk - sched.m_first)) { ok = false; break; }
                        fenced = true;
                    }
                    if (fenced) fence_proxy_async_global();
                }
                for (int it = 0; it < ti.k_iters; ++it) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                    const uint32_t fb_local = full_bar(s);
                    const uint32_t fb = map_to_cta(fb_local, 0);
                    if (cta == 0) mbar_expect_tx(fb_local, 2 * STAGE_TX);
                    const uint32_t a_dst = smem_base + s * DATA_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    const uint32_t sfa_dst = sf_base + s * SF_BYTES;
                    if (MODE == FMODE_WGRAD) {
                        const int kt = ti.k_tile0 + it;
                        const int brow = ti.n_blk * BN;
                        tma_load_2d_pair(a_dst, &tm.A, fb, kt * BKB, row0);
                        tma_load_2d_pair(b_dst, &tm.B, fb, kt * BKB, brow + static_cast<int>(cta) * 128);
                        tma_load_2d_pair(sfa_dst, &tm.SA, fb, 0, (row0 / 128) * p.a_ktiles + kt);
                        tma_load_2d_pair(sfa_dst + SF_TILE, &tm.SB, fb, 0, (brow / 128) * p.b_ktiles + kt);
                        tma_load_2d_pair(sfa_dst + 2 * SF_TILE, &tm.SB, fb, 0, (brow / 128 + 1) * p.b_ktiles + kt);
                    } else if (MODE == FMODE_FWD && ti.phase == 1) {
                        const int brow = ti.group * p.b3_rows_per_group + ti.n_blk * BN;
                        tma_load_2d_pair(a_dst, &tm.A2, fb, it * BKB, row0);
                        tma_load_2d_pair(sfa_dst, &tm.SA2, fb, 0, (row0 / 128) * p.a2_ktiles + it);
                        tma_load_2d_pair(b_dst, &tm.B3, fb, it * BKB, brow + static_cast<int>(cta) * 128);
                        tma_load_2d_pair(sfa_dst + SF_TILE, &tm.SB3, fb, 0, (brow / 128) * p.b3_ktiles + it);
                        tma_load_2d_pair(sfa_dst + 2 * SF_TILE, &tm.SB3, fb, 0, (brow / 128 + 1) * p.b3_ktiles + it);
                    } else {
                        const bool second = it >= kh;
                        const int kt = second ? it - kh : it;
                        const CUtensorMap* ta = second ? &tm.A2 : &tm.A;
                        const CUtensorMap* tsa = second ? &tm.SA2 : &tm.SA;
                        tma_load_2d_pair(a_dst, ta, fb, kt * BKB, row0);
                        tma_load_2d_pair(sfa_dst, tsa, fb, 0, (row0 / 128) * p.a_ktiles + kt);
                        if (kGateUp<MODE> || MODE == FMODE_FWD) {
                            const int brow = ti.group * p.b_rows_per_group + ti.n_blk * 128;
                            tma_load_2d_pair(b_dst, cta == 0 ? &tm.B : &tm.B2, fb, kt * BKB, brow);
                            tma_load_2d_pair(sfa_dst + SF_TILE, &tm.SB, fb, 0, (brow / 128) * p.b_ktiles + kt);
                            tma_load_2d_pair(sfa_dst + 2 * SF_TILE, &tm.SB2, fb, 0, (brow / 128) * p.b_ktiles + kt);
                        } else {
                            const CUtensorMap* tb = second ? &tm.B2 : &tm.B;
                            const CUtensorMap* tsb = second ? &tm.SB2 : &tm.SB;
                            const int brow = ti.group * p.b_rows_per_group + ti.n_blk * BN;
                            tma_load_2d_pair(b_dst, tb, fb, kt * BKB, brow + static_cast<int>(cta) * 128);
                            tma_load_2d_pair(sfa_dst + SF_TILE, tsb, fb, 0, (brow / 128) * p.b_ktiles + kt);
                            tma_load_2d_pair(sfa_dst + 2 * SF_TILE, tsb, fb, 0, (brow / 128 + 1) * p.b_ktiles + kt);
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA)
        if (lane == 0 && cta == 0) {
            // block-scaled instruction descriptor: E4M3 x E4M3, E8M0 scales, M = 256 over the pair, N = 256
            constexpr uint32_t idesc0 = (static_cast<uint32_t>(BN >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(TILE_M >> 4) << 24);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int local = 0;
            Tile next_ti = {};
            if (tile_id0 < sched.total) next_ti = sched.get(p, tile_id0);
            for (int t = tile_id0; ok && t < sched.total; t += tile_stride, ++local) {
                const Tile ti = next_ti;
                if (t + tile_stride < sched.total) next_ti = sched.get(p, t + tile_stride);
                if (!mbar_wait(tempty_bar, (local & 1) ^ 1u, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base;
                for (int it = 0; it < ti.k_iters; ++it) {
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * DATA_BYTES;
                    const uint32_t b_addr = a_addr + A_BYTES;
                    const uint32_t sf_addr = sf_base + s * SF_BYTES;
                    const uint32_t sf_cols = tmem_base + SF_COL0 + (s & 1) * SF_SET_COLS;
                    tmem_cp_32x128b_warpx4_pair(sf_cols, make_smem_desc_plain16(sf_addr));
                    tmem_cp_32x128b_warpx4_pair(sf_cols + 4, make_smem_desc_plain16(sf_addr + SF_TILE));
                    tmem_cp_32x128b_warpx4_pair(sf_cols + 8, make_smem_desc_plain16(sf_addr + 2 * SF_TILE));
                    const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
                    const uint64_t b_desc = make_smem_desc(b_addr, 16, 1024);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t idesc = idesc0 | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29);
                        umma_mxf8_pair(d_tmem, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2), idesc,
                                       sf_cols, sf_cols + 4, (it | k) != 0 ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar(s), 0x3);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar, 0x3);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        // warp w drains lanes 32*(w%4).. (the quarter of tensor memory it may read), columns 128*half..
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_tile = static_cast<int>(cta) * 128 + quarter * 32 + lane;
        int local = 0;
        bool ok = true;
        for (int t = tile_id0; ok && t < sched.total; t += tile_stride, ++local) {
            const Tile ti = sched.get(p, t);
            if (!mbar_wait(tfull_bar, local & 1, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
            tc_fence_after();
            if (MODE == FMODE_GATEUP_QUANT || (MODE == FMODE_FWD && ti.phase == 0)) {
                // This warp: 32 rows (its lanes) x gate columns [64 half, +64) and the matching up columns of the tile.
                const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
                uint32_t gw[32], uw[32];                    // bf16 pairs: the values the bf16 path would have stored
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(t_lane + half * 64 + c * 32, r0);
                    tmem_ld_32x32(t_lane + 128 + half * 64 + c * 32, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        gw[c * 16 + i] = pack_bf16(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
                        uw[c * 16 + i] = pack_bf16(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar, 0));

                const int64_t row = static_cast<int64_t>(ti.m_blk) * TILE_M + row_in_tile;
                const int64_t col0 = static_cast<int64_t>(ti.n_blk) * 128 + half * 64;
                const int64_t N = p.N;
                // along columns: this thread owns two whole 32-column blocks of its row in each tensor
                quantize_row_blocks(gw, p.gate_q, p.gate_sc, row, col0, N);
                quantize_row_blocks(uw, p.up_q, p.up_sc, row, col0, N);
                // hidden only now: gate and up die pair by pair as it is computed (96 live values would not fit)
                uint32_t hw[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float g0 = bf16_lo(gw[i]), g1 = bf16_hi(gw[i]), u0 = bf16_lo(uw[i]), u1 = bf16_hi(uw[i]);
                    if (p.has_limit) {
                        g0 = fminf(g0, p.limit);
                        g1 = fminf(g1, p.limit);
                        u0 = fminf(fmaxf(u0, -p.limit), p.limit);
                        u1 = fminf(fmaxf(u1, -p.limit), p.limit);
                    }
                    hw[i] = pack2(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
                }
                quantize_row_blocks(hw, p.hid_q, p.hid_sc, row, col0, N);
                // along tokens: the warp's 32 lanes are one 32-token block of each of its 64 columns
                const int64_t row_blk0 = static_cast<int64_t>(ti.m_blk) * TILE_M + static_cast<int>(cta) * 128 + quarter * 32;
                uint32_t my_scales = 0u;                    // lane j keeps the two scale bytes of column pair j
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    uint32_t m = hw[j] & 0x7fff7fffu;
#pragma unroll
                    for (int d = 16; d >= 1; d >>= 1) m = absmax2(m, __shfl_xor_sync(0xffffffffu, m, d));
                    float inv_a, inv_b;
                    const uint32_t byte_a = scale_byte(bf16_lo(m), &inv_a);
                    const uint32_t byte_b = scale_byte(bf16_hi(m), &inv_b);
                    uint16_t pair;
                    asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(pair) : "f"(bf16_lo(hw[j]) * inv_a), "f"(bf16_hi(hw[j]) * inv_b));
                    const int64_t col = col0 + 2 * j;
                    p.hid_qt[col * p.t_rows + row] = static_cast<uint8_t>(pair & 0xffu);
                    p.hid_qt[(col + 1) * p.t_rows + row] = static_cast<uint8_t>(pair >> 8);
                    if (lane == j) my_scales = byte_a | (byte_b << 8);
                }
                {
                    const int64_t col = col0 + 2 * lane;
                    p.hid_sct[scale_offset(col, row_blk0 >> 5, p.t_rows >> 7)] = static_cast<uint8_t>(my_scales & 0xffu);
                    p.hid_sct[scale_offset(col + 1, row_blk0 >> 5, p.t_rows >> 7)] = static_cast<uint8_t>(my_scales >> 8);
                }
                if (MODE == FMODE_FWD) {      // this warp's part of the hidden rows is stored: count it for the down tiles
                    __syncwarp();
                    if (lane == 0) red_release_gpu_add(p.blk_done + (ti.m_blk - sched.m_first), 1);
                }
                continue;
            }
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(half * 128);
            const bool empty_k = ti.k_iters == 0;
            // drain this warp's part of the accumulator into registers as packed bf16, then hand it back to the MMA lane
            const int tile_row = ti.m_blk * TILE_M + row_in_tile;
            bool row_ok = true;
            size_t row = static_cast<size_t>(tile_row);
            __nv_bfloat16* dst;
            int cols_left = 128;
            if (MODE == FMODE_DUALB) {
                dst = (half ? p.D2 : p.D) + row * p.ldd + static_cast<size_t>(ti.n_blk) * 128;
            } else {
                if (MODE == FMODE_WGRAD) {
                    row_ok = tile_row < p.M;
                    row += static_cast<size_t>(ti.group) * p.M;
                }
                dst = p.D + row * p.ldd + static_cast<size_t>(ti.n_blk) * BN + half * 128;
                cols_left = (MODE == FMODE_FWD ? p.N2 : p.N) - ti.n_blk * BN - half * 128;
                if (p.D == nullptr) row_ok = false;        // pushed only
            }
            __nv_bfloat16* pdst = nullptr;                 // this row's place in its home rank's buffer
            if ((MODE == FMODE_NT || MODE == FMODE_FWD) && p.push) {
                const int pr = p.push_rank[tile_row];
                if (pr >= 0 && pr < p.push_ranks &&
                    index_ok(IndexGuard{p.push_limit, p.status}, p.push_idx[tile_row], kBadIndexGemmPush, tile_row)) {
                    const size_t slot = static_cast<size_t>(p.push_idx[tile_row]);
                    pdst = static_cast<__nv_bfloat16*>(p.push_dst.p[pr]) + slot * p.ldd + static_cast<size_t>(ti.n_blk) * BN + half * 128;
                    if (p.push_values && ti.n_blk == 0 && half == 0) static_cast<float*>(p.push_val.p[pr])[slot] = p.push_values[tile_row];
                }
            }
            const bool add_old = MODE == FMODE_WGRAD && p.accumulate;
            if (add_old && empty_k) row_ok = false;        // nothing to add: the stored gradient stays
            uint32_t packed[64];
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
                uint32_t r0[32], r1[32];
                tmem_ld_32x32(t_addr + c * 32, r0);
                tmem_ld_32x32(t_addr + c * 32 + 32, r1);
                tmem_ld_wait();
                if (add_old && row_ok && c * 32 < cols_left) {      // fp32 accumulator + stored bf16, rounded once
                    const uint32_t* old0 = reinterpret_cast<const uint32_t*>(dst + c * 32);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 f0 = unpack_bf16(old0[i]), f1 = unpack_bf16(old0[16 + i]);
                        r0[2 * i] = __float_as_uint(__uint_as_float(r0[2 * i]) + f0.x);
                        r0[2 * i + 1] = __float_as_uint(__uint_as_float(r0[2 * i + 1]) + f0.y);
                        r1[2 * i] = __float_as_uint(__uint_as_float(r1[2 * i]) + f1.x);
                        r1[2 * i + 1] = __float_as_uint(__uint_as_float(r1[2 * i + 1]) + f1.y);
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    packed[c * 16 + i] = empty_k ? 0u : pack_bf16(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
                    packed[c * 16 + 16 + i] = empty_k ? 0u : pack_bf16(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar, 0));

            if (row_ok) {
                if (p.wide_stores) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (q * 16 < cols_left) st_global_v8(dst + 16 * q, &packed[8 * q]);
                } else {
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        if (q * 8 < cols_left)
                            st_global_v4(dst + 8 * q, packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            if ((MODE == FMODE_NT || MODE == FMODE_FWD) && p.push) {
                // Rows that go to a peer cross NVLink: 32 rows x 32 columns at a time are transposed through shared memory
                // so that four lanes store 64 contiguous bytes of a row (two stores fill a 128-byte line) instead of every
                // lane storing 32 bytes of a row of its own.  Whole warp; rows without a home have a null pointer.
                const uint32_t stage = bars + 256u + static_cast<uint32_t>(warp - 2) * 2048u;
                const unsigned long long own_home = reinterpret_cast<unsigned long long>(pdst);
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    if (st * 32 >= cols_left) break;
                    __syncwarp();             // the previous piece has been read out of the buffer
#pragma unroll
                    for (int u = 0; u < 4; ++u)      // row `lane`, 16-byte unit u at u ^ ((lane >> 1) & 3): conflict-free both ways
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 64u + static_cast<uint32_t>((u ^ ((lane >> 1) & 3)) << 4)),
                                     "r"(packed[16 * st + 4 * u]), "r"(packed[16 * st + 4 * u + 1]), "r"(packed[16 * st + 4 * u + 2]),
                                     "r"(packed[16 * st + 4 * u + 3]) : "memory");
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = 8 * i + (lane >> 2), unit = lane & 3;
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                     : "r"(stage + rr * 64u + static_cast<uint32_t>((unit ^ ((rr >> 1) & 3)) << 4)) : "memory");
                        __nv_bfloat16* home = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, own_home, rr));
                        if (home) st_global_v4(home + st * 32 + unit * 8, v0, v1, v2, v3);
                    }
                }
            }
            if (MODE == FMODE_FWD && p.win_done) {
                __syncwarp();
                if (lane == 0) red_release_gpu_add(p.win_done + ti.window, 1);
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <int MODE>
int launch(const Maps& m, const FParams& p, int tiles_upper_bound, cudaStream_t stream) {
    MOKB_CUDA(cudaFuncSetAttribute(grouped_gemm_mxfp8_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    int pairs = sm_count() / 2;
    // a launch that waits for another kernel's rows leaves one pair of SMs to that kernel (see gemm.cu)
    if (p.win_ready) pairs -= p.reserve_pairs < pairs - 1 ? p.reserve_pairs : pairs - 1;
    if (tiles_upper_bound < pairs) pairs = tiles_upper_bound;
    if (pairs < 1) return MOKB_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(pairs * 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MOKB_CUDA(cudaLaunchKernelEx(&cfg, grouped_gemm_mxfp8_kernel<MODE>, m, p));
    note_launch();
    return MOKB_OK;
}

int data_map(CUtensorMap* out, const void* base, uint64_t k, uint64_t rows) {
    return make_tmap_2d(out, base, 1, k, rows, k, 128, 128);
}
int scale_map(CUtensorMap* out, const void* base, uint64_t tiles) {
    return make_tmap_2d(out, base, 4, 128, tiles, 512, 128, 1);
}

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" int mokb_grouped_gemm_mxfp8(const mokb_gemm_fp8_args* g, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_REQUIRE(g != nullptr, "grouped_gemm_mxfp8: null args");
    static const char* const kTags[5] = {"gemm_mxfp8_nt", "gemm_mxfp8_gate_up", "gemm_mxfp8_wgrad", "gemm_mxfp8_gate_up_swiglu_quant",
                                         "gemm_mxfp8_fwd_routed"};
    TraceScope trace(stream, kTags[g->mode >= 0 && g->mode <= 4 ? g->mode : 0], g->row_begin);
    MOKB_REQUIRE(g->mode >= 0 && g->mode <= 4, "grouped_gemm_mxfp8: unknown mode %d", g->mode);
    MOKB_REQUIRE(g->A && g->A_sc && g->B && g->B_sc && g->status, "grouped_gemm_mxfp8: null pointer");
    MOKB_REQUIRE(g->D || g->mode == FMODE_GATEUP_QUANT || g->mode == FMODE_FWD || (g->mode == FMODE_NT && g->push_ptrs_host),
                 "grouped_gemm_mxfp8: D may only be left out when the result is pushed to peers");
    MOKB_REQUIRE(g->G >= 1 && g->ldd % 8 == 0, "grouped_gemm_mxfp8: bad G or ldd");
    MOKB_REQUIRE(g->rows_static > 0 && g->rows_static % 256 == 0, "grouped_gemm_mxfp8: rows must be a positive multiple of 256");
    FParams p;
    memset(&p, 0, sizeof(p));
    p.rows_cap = g->rows_static;
    p.row_begin = g->row_begin;
    p.row_end = g->row_end > 0 ? g->row_end : g->rows_static;
    MOKB_REQUIRE(p.row_begin >= 0 && p.row_begin % 256 == 0 && p.row_end % 256 == 0 && p.row_begin <= p.row_end && p.row_end <= g->rows_static,
                 "grouped_gemm_mxfp8: bad row window");
    p.num_rows = g->num_rows;
    p.group_of_block = g->group_of_block;
    p.group_offsets = g->group_offsets;
    p.G = g->G; p.M = g->M; p.N = g->N; p.K = g->K;
    p.D = static_cast<__nv_bfloat16*>(g->D);
    p.D2 = static_cast<__nv_bfloat16*>(g->D2);
    p.ldd = g->ldd;
    p.wide_stores = g->ldd % 16 == 0 && reinterpret_cast<uintptr_t>(g->D) % 32 == 0 && reinterpret_cast<uintptr_t>(g->D2) % 32 == 0;
    p.status = g->status;
    if (g->push_ptrs_host) {
        MOKB_REQUIRE(g->mode == FMODE_NT || g->mode == FMODE_FWD, "grouped_gemm_mxfp8: push is for modes 0 and 4");
        MOKB_REQUIRE(g->push_ep_size >= 1 && g->push_ep_size <= MOKB_MAX_EP && g->push_rank && g->push_idx, "grouped_gemm_mxfp8: push needs ranks and indices");
        MOKB_REQUIRE((g->push_values == nullptr) == (g->push_value_ptrs_host == nullptr), "grouped_gemm_mxfp8: push_values and push_value_ptrs_host go together");
        MOKB_REQUIRE(g->push_index_limit >= 0 && g->push_index_limit <= INT32_MAX, "grouped_gemm_mxfp8: push_index_limit must fit 31 bits");
        p.push_limit = static_cast<int>(g->push_index_limit);
        p.push = 1; p.push_ranks = g->push_ep_size; p.push_rank = g->push_rank; p.push_idx = g->push_idx; p.push_values = g->push_values;
        p.push_wide = g->ldd % 16 == 0;
        for (int r = 0; r < kPeerMax; ++r) p.push_dst.p[r] = p.push_val.p[r] = nullptr;
        for (int r = 0; r < g->push_ep_size; ++r) {
            MOKB_REQUIRE(g->push_ptrs_host[r] != 0 && (g->push_ptrs_host[r] & 15) == 0, "grouped_gemm_mxfp8: push pointer of rank %d is null or not 16-byte aligned", r);
            p.push_dst.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(g->push_ptrs_host[r]));
            if ((g->push_ptrs_host[r] & 31) != 0) p.push_wide = 0;
            if (g->push_value_ptrs_host) {
                MOKB_REQUIRE(g->push_value_ptrs_host[r] != 0, "grouped_gemm_mxfp8: push value pointer of rank %d is null", r);
                p.push_val.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(g->push_value_ptrs_host[r]));
            }
        }
    }
    if (g->mode != FMODE_WGRAD) {
        MOKB_REQUIRE(g->window_rows >= 0 && g->window_rows % 256 == 0, "grouped_gemm_mxfp8: window_rows must be a multiple of 256");
        MOKB_REQUIRE(g->win_ready == nullptr || (g->window_rows > 0 && g->win_ready_target > 0), "grouped_gemm_mxfp8: win_ready needs window_rows and a target");
        p.window_rows = g->window_rows;
        p.win_ready = g->win_ready;
        p.win_ready_target = g->win_ready_target;
        MOKB_REQUIRE(g->reserve_sms >= 0, "grouped_gemm_mxfp8: reserve_sms must not be negative");
        p.reserve_pairs = g->reserve_sms > 0 ? (g->reserve_sms + 1) / 2 : 1;
    }
    Maps m;
    memset(&m, 0, sizeof(m));
    const uint64_t rows = static_cast<uint64_t>(g->rows_static);
    const int m_tiles = (p.row_end - p.row_begin) / TILE_M;
    if (g->mode == FMODE_WGRAD) {
        // A [M, rows], B [N, rows]: the contraction runs over the token axis, one window per group
        MOKB_REQUIRE(g->M > 0 && g->M % 128 == 0 && g->N > 0 && g->N % 128 == 0, "grouped_gemm_mxfp8 WGRAD: M and N must be multiples of 128");
        MOKB_REQUIRE(g->group_offsets != nullptr, "grouped_gemm_mxfp8 WGRAD: group_offsets required");
        MOKB_REQUIRE(g->t_first >= 0 && g->t_first % 128 == 0, "grouped_gemm_mxfp8 WGRAD: t_first must be a non-negative multiple of 128");
        MOKB_TRY(data_map(&m.A, g->A, rows, g->M));
        MOKB_TRY(data_map(&m.B, g->B, rows, g->N));
        MOKB_TRY(scale_map(&m.SA, g->A_sc, static_cast<uint64_t>(g->M / 128) * (rows / 128)));
        MOKB_TRY(scale_map(&m.SB, g->B_sc, static_cast<uint64_t>(g->N / 128) * (rows / 128)));
        m.A2 = m.A; m.B2 = m.B; m.SA2 = m.SA; m.SB2 = m.SB;
        p.a_ktiles = p.b_ktiles = static_cast<int>(rows / 128);
        p.k_tile_origin = g->t_first / BKB;
        p.accumulate = g->accumulate;
        return launch<FMODE_WGRAD>(m, p, g->G * ((g->M + TILE_M - 1) / TILE_M) * ((g->N + BN - 1) / BN), stream);
    }
    MOKB_REQUIRE(g->K > 0 && g->K % 128 == 0 && g->N > 0 && g->N % 128 == 0, "grouped_gemm_mxfp8: K and N must be multiples of 128");
    const uint64_t brows = static_cast<uint64_t>(g->G) * g->N;
    MOKB_TRY(data_map(&m.A, g->A, g->K, rows));
    MOKB_TRY(data_map(&m.B, g->B, g->K, brows));
    MOKB_TRY(scale_map(&m.SA, g->A_sc, (rows / 128) * (g->K / 128)));
    MOKB_TRY(scale_map(&m.SB, g->B_sc, (brows / 128) * (g->K / 128)));
    m.A2 = m.A; m.B2 = m.B; m.SA2 = m.SA; m.SB2 = m.SB; m.B3 = m.B; m.SB3 = m.SB;
    p.a_ktiles = p.b_ktiles = g->K / 128;
    p.b_rows_per_group = g->N;
    if (g->mode == FMODE_DUALB || g->mode == FMODE_GATEUP_QUANT || g->mode == FMODE_FWD) {
        MOKB_REQUIRE(g->B2 && g->B2_sc, "grouped_gemm_mxfp8 gate/up: B2 and B2_sc required");
        MOKB_TRY(data_map(&m.B2, g->B2, g->K, brows));
        MOKB_TRY(scale_map(&m.SB2, g->B2_sc, (brows / 128) * (g->K / 128)));
        if (g->mode == FMODE_DUALB) {
            MOKB_REQUIRE(g->D2 != nullptr, "grouped_gemm_mxfp8 mode 1: D2 required");
            return launch<FMODE_DUALB>(m, p, m_tiles * (g->N / 128), stream);
        }
        MOKB_REQUIRE(g->gate_q && g->gate_sc && g->up_q && g->up_sc && g->hid_q && g->hid_sc && g->hid_qt && g->hid_sct,
                     "grouped_gemm_mxfp8 mode 3: all eight quantised outputs required");
        MOKB_REQUIRE(g->t_rows > 0 && g->t_rows % 128 == 0, "grouped_gemm_mxfp8 mode 3: t_rows must be a positive multiple of 128");
        MOKB_REQUIRE(((reinterpret_cast<uintptr_t>(g->gate_q) | reinterpret_cast<uintptr_t>(g->up_q) | reinterpret_cast<uintptr_t>(g->hid_q)) & 31) == 0,
                     "grouped_gemm_mxfp8 mode 3: quantised outputs must be 32-byte aligned");
        p.gate_q = static_cast<uint8_t*>(g->gate_q); p.gate_sc = static_cast<uint8_t*>(g->gate_sc);
        p.up_q = static_cast<uint8_t*>(g->up_q); p.up_sc = static_cast<uint8_t*>(g->up_sc);
        p.hid_q = static_cast<uint8_t*>(g->hid_q); p.hid_sc = static_cast<uint8_t*>(g->hid_sc);
        p.hid_qt = static_cast<uint8_t*>(g->hid_qt); p.hid_sct = static_cast<uint8_t*>(g->hid_sct);
        p.t_rows = g->t_rows;
        p.has_limit = g->has_swiglu_limit;
        p.limit = g->swiglu_limit;
        if (g->mode == FMODE_FWD) {
            MOKB_REQUIRE(g->blk_done != nullptr, "grouped_gemm_mxfp8 mode 4: blk_done required");
            MOKB_REQUIRE(g->N2 >= 0 && g->N2 % BN == 0, "grouped_gemm_mxfp8 mode 4: N2 must be a multiple of 256");
            p.blk_done = g->blk_done;
            p.win_done = g->win_done;
            if (g->N2 > 0) {
                // the down projection reads the hidden rows this launch writes: A2 = hid_q [rows, N], contraction over N
                MOKB_REQUIRE(g->B3 && g->B3_sc && (g->D || g->push_ptrs_host), "grouped_gemm_mxfp8 mode 4: B3, B3_sc and D (or push pointers) required");
                const uint64_t b3rows = static_cast<uint64_t>(g->G) * g->N2;
                MOKB_TRY(data_map(&m.A2, g->hid_q, g->N, rows));
                MOKB_TRY(scale_map(&m.SA2, g->hid_sc, (rows / 128) * (g->N / 128)));
                MOKB_TRY(data_map(&m.B3, g->B3, g->N, b3rows));
                MOKB_TRY(scale_map(&m.SB3, g->B3_sc, (b3rows / 128) * (g->N / 128)));
                p.N2 = g->N2; p.K2 = g->N; p.b3_rows_per_group = g->N2;
                p.a2_ktiles = p.b3_ktiles = g->N / 128;
            }
            return launch<FMODE_FWD>(m, p, m_tiles * (g->N / 128 + g->N2 / BN), stream);
        }
        return launch<FMODE_GATEUP_QUANT>(m, p, m_tiles * (g->N / 128), stream);
    }
    if (g->A2) {
        MOKB_REQUIRE(g->A2_sc && g->B2 && g->B2_sc, "grouped_gemm_mxfp8: the second operand pair needs data and scales");
        MOKB_TRY(data_map(&m.A2, g->A2, g->K, rows));
        MOKB_TRY(data_map(&m.B2, g->B2, g->K, brows));
        MOKB_TRY(scale_map(&m.SA2, g->A2_sc, (rows / 128) * (g->K / 128)));
        MOKB_TRY(scale_map(&m.SB2, g->B2_sc, (brows / 128) * (g->K / 128)));
        p.dual = 1;
    }
    return launch<FMODE_NT>(m, p, m_tiles * ((g->N + BN - 1) / BN), stream);
}
