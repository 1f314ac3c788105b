// Grouped BF16 GEMM for the expert FFN, forward and backward, on the 5th-gen
// tensor cores: tcgen05.mma with the fp32 accumulator in tensor memory, operands
// staged in 128B-swizzled shared memory by TMA, and persistent, warp-specialised
// CTAs.
//
//   warp 0      TMA producer   (one lane)  : global -> smem ring
//   warp 1      MMA issuer     (one lane)  : 4 x tcgen05.mma (K = 16 each) per 64-wide K stage
//   warps 2..5  epilogue                   : TMEM -> registers -> bf16 -> global
//
// Two tile shapes share the code (template parameter NCTA):
//   NCTA = 2  a pair of CTAs on neighbouring SMs (cluster of 2, tcgen05 cta_group::2) computes a
//             256 x 256 tile.  Each CTA stages 128 rows of A and 128 of the 256 B columns
//             (32 KB per stage, 6 stages), the even CTA issues 256 x 256 x 16 MMAs that read both
//             CTAs' shared memory, and each CTA holds and drains its own 128 rows of the
//             accumulator.  Per SM this needs a third less operand traffic than a 128 x 256
//             tile per CTA, which is what bounds the single-CTA form.  Every CTA loads only its
//             own half-tiles; barriers are signalled across the pair.
//   NCTA = 1  one CTA per 128 x 256 tile (48 KB per stage, 4 stages).
// The 512 TMEM columns hold two accumulators, so the epilogue of tile i overlaps the main loop
// of tile i+1 (the reference keeps a single accumulator per CTA, csrc/megakernel/forward.cuh:84).
//
// One kernel template covers the operand layouts the layer needs
// (reference: csrc/megakernel/grouped_gemm.cuh:1-381):
//   MODE_NT      D[rows,N] = A[rows,K] * W[g][N,K]^T                 (down projection)
//   MODE_SWIGLU  gate,up = A * Wg[g]^T, A * Wu[g]^T; hidden = SwiGLU  (one 128+128 column tile)
//   MODE_NN      D[rows,N] = A[rows,K] * W[g][K,N] (+ A2 * W2[g])    (input gradients)
//   MODE_WGRAD   D[g][M,N] = A[rows_g,M]^T * B[rows_g,N]             (weight gradients)
//   MODE_FWD     MODE_SWIGLU tiles and the MODE_NT (down) tiles of the same rows in ONE persistent launch,
//                window by window (a window = the rows one dispatch launch pulls): the task loop of the
//                reference's forward megakernel (csrc/megakernel/forward.cuh:146-266) with its global-memory
//                counters (csrc/megakernel/utils.cuh:1-13), every wait bounded.
// Expert segments are multiples of 256 rows, so a tile never straddles two experts.
//
// Counters (row-tiled modes, all optional): `win_ready[w]` is raised by the dispatch blocks of window w and
// awaited by the TMA producer before it loads the first A rows of that window; MODE_FWD also counts the
// epilogue warps that finished the gate/up tiles of a 256-row block (`blk_done`, awaited before a down tile
// loads `hidden`) and those that finished the down tiles of a window (`win_done`, awaited by the combine
// kernel).  Producers publish with a release at GPU scope after their stores; the consumer acquires and then
// orders the generic-proxy writes before its own TMA reads with a proxy fence.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace mokb {
namespace {

constexpr int BN = 256, BK = 64;
constexpr int A_BYTES = 128 * BK * 2;           // 16 KB: 128 rows (or 2 x 64 columns) of A per CTA
constexpr int CHUNK_BYTES = 64 * BK * 2;        // one 64-wide MN-major chunk: 8 KB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_ROWS = 1024;                // rows per raster super-group

enum { MODE_NT = 0, MODE_SWIGLU = 1, MODE_NN = 2, MODE_WGRAD = 3, MODE_FWD = 4 };

template <int NCTA>
struct Geo {
    static constexpr int TILE_M = 128 * NCTA;
    static constexpr int B_COLS = BN / NCTA;                 // B columns staged by one CTA
    static constexpr int B_BYTES = B_COLS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;    // 48 KB / 32 KB
    static constexpr int STAGES = NCTA == 2 ? 6 : 4;
    static constexpr int GROUP_M = GROUP_ROWS / TILE_M;
    // + one 4 KB transposition buffer per epilogue warp (32 rows x 128 bytes)
    static constexpr size_t SMEM_BYTES = static_cast<size_t>(STAGES) * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + 4 * 4096;
};

struct KParams {
    int rows_cap;                    // static upper bound of rows
    int row_begin, row_end;          // row window (multiples of 256); row_end <= rows_cap
    const int32_t* num_rows;         // device, optional
    const int32_t* group_of_block;   // device [rows/128], optional
    const int32_t* group_offsets;    // device [G+1], MODE_WGRAD
    const int32_t* group_k_end;      // device [G], MODE_WGRAD, optional: rows of group g from here on are zero in both operands
    int G, M, N, K;
    int b_rows_per_group;            // rows of the flattened weight tensor per group
    int dual;                        // MODE_NN: second (A2, B2) pair accumulates into the same tile
    __nv_bfloat16 *D, *D2, *D3;
    int ldd;
    int wide_stores;                 // output rows are 32-byte aligned: the epilogue stores 32 bytes per instruction
    int has_limit;
    float limit;
    int accumulate;                  // MODE_WGRAD: add to the stored bf16 result instead of overwriting it
    // counters (see the top of the file)
    int window_rows;                 // rows per window, a multiple of 256; 0 = one window
    const int32_t* win_ready;        // [windows from row_begin], optional
    int win_ready_target;
    // MODE_FWD: the down projection that follows gate/up + SwiGLU
    int N2, K2;                      // down: N2 = hidden columns (multiple of 256; 0 = no down tiles), K2 = contraction
    int b3_rows_per_group;
    __nv_bfloat16* D4;
    int ldd4;
    int32_t* blk_done;               // [256-row blocks from row_begin]
    int32_t* win_done;               // [windows from row_begin], optional
    // push (MODE_NT, MODE_NN, the down tiles of MODE_FWD): row r of the result goes to row push_idx[r] of rank
    // push_rank[r]'s buffer (rows with a rank outside [0, push_ranks) go nowhere) -- combine without a combine kernel
    int push, push_ranks, push_wide, push_limit;
    const int32_t* push_rank;
    const int32_t* push_idx;
    const float* push_values;        // optional: push_val[rank][idx] = push_values[r], written with the first column tile
    int32_t* status;
    int line_stores;                 // the epilogue transposes through shared memory and stores whole 128-byte lines
    PeerPtrs push_dst, push_val;
};

struct Tile {
    int m_blk, n_blk, group, k_iters, k_row0;
    int phase;                       // MODE_FWD: 0 = gate/up + SwiGLU tile, 1 = down tile
    int window;                      // window of the tile's rows, counted from row_begin
};

template <int MODE, int NCTA>
struct Sched {
    int m_blocks, n_blocks, total, m_first;
    int n_gu, n_nt, win_blocks;      // MODE_FWD: column tiles of the two phases; row tiles per window (all row-tiled modes)
    __device__ Sched(const KParams& p) {
        m_first = 0;
        n_gu = n_nt = 0;
        win_blocks = 1 << 30;
        constexpr int TM = Geo<NCTA>::TILE_M;
        if (MODE == MODE_WGRAD) {
            m_blocks = (p.M + TM - 1) / TM;
            n_blocks = (p.N + BN - 1) / BN;
            total = p.G * m_blocks * n_blocks;
            // accumulating over no rows at all (an empty macrobatch) leaves every gradient as it is: no tiles
            if (p.accumulate && p.group_offsets[p.G] == p.group_offsets[0]) total = 0;
        } else {
            int rows = p.num_rows ? *p.num_rows : p.rows_cap;
            if (rows < 0) rows = 0;                 // the row window below never exceeds the tensors (row_end <= rows_cap)
            const int hi = min(rows, p.row_end), lo = min(p.row_begin, hi);
            m_first = lo / TM;
            m_blocks = (hi - lo) / TM;
            n_blocks = MODE == MODE_SWIGLU ? p.N / 128 : (p.N + BN - 1) / BN;
            total = m_blocks * n_blocks;
            if (p.window_rows > 0) win_blocks = p.window_rows / TM;
            if (MODE == MODE_FWD) {
                n_gu = p.N / 128;
                n_nt = p.N2 / BN;
                total = m_blocks * (n_gu + n_nt);
            }
        }
    }
    __device__ Tile get(const KParams& p, int t) const {
        constexpr int TM = Geo<NCTA>::TILE_M;
        constexpr int GM = Geo<NCTA>::GROUP_M;
        Tile ti;
        if (MODE == MODE_WGRAD) {
            const int per = m_blocks * n_blocks;
            ti.group = t / per;
            const int rem = t - ti.group * per;
            ti.n_blk = rem / m_blocks;
            ti.m_blk = rem - ti.n_blk * m_blocks;
            ti.k_row0 = p.group_offsets[ti.group];
            int k_end = p.group_offsets[ti.group + 1];
            if (p.group_k_end) k_end = min(k_end, max(p.group_k_end[ti.group], ti.k_row0));
            ti.k_iters = (k_end - ti.k_row0 + BK - 1) / BK;      // a partial last stage reads rows that are zero
        } else if (MODE == MODE_FWD) {
            // window by window: all gate/up tiles of the window's rows, then all their down tiles; inside a phase,
            // super-groups of 1024 rows x every column tile
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
            const int per = GM * nb;
            const int sg = local / per;
            const int first = sg * GM;
            const int gsize = min(GM, wc - first);
            const int in = local - sg * per;
            ti.n_blk = in / gsize;
            ti.m_blk = m_first + blk0 + first + (in - ti.n_blk * gsize);
            ti.window = w;
            ti.group = p.group_of_block ? p.group_of_block[ti.m_blk * (TM / 128)] : 0;
            ti.k_row0 = 0;
            ti.k_iters = (ti.phase ? p.K2 : p.K) / BK;
        } else {
            const int per = GM * n_blocks;
            const int sg = t / per;
            const int first = sg * GM;
            const int gsize = min(GM, m_blocks - first);
            const int in = t - sg * per;
            ti.n_blk = in / gsize;
            ti.m_blk = m_first + first + (in - ti.n_blk * gsize);
            ti.group = p.group_of_block ? p.group_of_block[ti.m_blk * (TM / 128)] : 0;
            ti.k_row0 = 0;
            ti.k_iters = (p.K / BK) * (p.dual ? 2 : 1);
            ti.phase = 0;
            ti.window = (ti.m_blk - m_first) / win_blocks;
        }
        return ti;
    }
};

__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 32 fp32 accumulator columns of one row -> 32 bf16 (64 bytes) in global memory; `wide`: the row is 32-byte
// aligned, so two 32-byte stores (one full sector each) replace four 16-byte ones
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const uint32_t (&r)[32], bool wide) {
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    if (wide) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * q), "r"(w[8 * q]), "r"(w[8 * q + 1]),
                         "r"(w[8 * q + 2]), "r"(w[8 * q + 3]), "r"(w[8 * q + 4]), "r"(w[8 * q + 5]), "r"(w[8 * q + 6]), "r"(w[8 * q + 7])
                         : "memory");
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) st_global_v4(dst + 8 * q, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
}

template <int NCTA>
__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* t, uint32_t bar, int c0, int c1) {
    if (NCTA == 2) tma_load_2d_pair(dst, t, bar, c0, c1);
    else tma_load_2d(dst, t, bar, c0, c1);
}

// 128 registers per thread at most: registers are handed out per SM quarter (16 K each), a CTA's six warps put two
// on a quarter, and the dispatch / quantise blocks that run beside the GEMM (eight warps of 56 registers, two per
// quarter) must still fit there -- a GEMM that waits for their rows on an SM they cannot enter would wait for ever.
template <int MODE, int NCTA>
__global__ void __maxnreg__(128)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                    const __grid_constant__ CUtensorMap tmB3, const KParams p) {
    using G = Geo<NCTA>;
    constexpr int STAGES = G::STAGES;
    constexpr int STAGE_BYTES = G::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + STAGES * STAGE_BYTES;
    // barrier block: full[S] | empty[S] | tmem_full[2] | tmem_empty[2] | tmem_ptr | abort
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    uint8_t* bar_gen = smem_gen + STAGES * STAGE_BYTES;
    volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 8 * (2 * STAGES + 4) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta = NCTA == 2 ? cluster_ctarank() : 0u;     // 0 = leader of the pair
    const int tile_id0 = NCTA == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int tile_stride = NCTA == 2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);        // leader's: one arrive.expect_tx by the leader's producer + all TMA bytes
            mbar_init(empty_bar(s), 1);       // one commit arrival per use (sent to both CTAs of a pair)
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4 * NCTA);   // leader's: one arrival per epilogue warp of the pair
        }
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (MODE == MODE_SWIGLU || MODE == MODE_FWD || (MODE == MODE_NN && p.dual)) {
            tma_prefetch_desc(&tmB2);
            if (MODE == MODE_NN) tma_prefetch_desc(&tmA2);
        }
        if (MODE == MODE_FWD && p.N2 > 0) {
            tma_prefetch_desc(&tmA2);
            tma_prefetch_desc(&tmB3);
        }
    }
    if (warp == 1) {
        if (NCTA == 2) {
            tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), TMEM_COLS);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (NCTA == 2) cluster_sync_all();     // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_slot;

    const Sched<MODE, NCTA> sched(p);

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs of a pair)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            const int kh = p.K / BK;
            int waited_window = -1;
            // the next tile's coordinates (integer divisions, loads of the group tables) are worked out while this
            // tile's stages are in flight: with a short contraction the look-up would otherwise stall every tile
            Tile next_ti = {};
            if (tile_id0 < sched.total) next_ti = sched.get(p, tile_id0);
            for (int t = tile_id0; ok && t < sched.total; t += tile_stride) {
                const Tile ti = next_ti;
                if (t + tile_stride < sched.total) next_ti = sched.get(p, t + tile_stride);
                const int row0 = ti.m_blk * G::TILE_M + static_cast<int>(cta) * 128;    // this CTA's rows of A / D
                if (MODE != MODE_WGRAD) {
                    // rows that another kernel (or, for a down tile, other CTAs of this one) is still producing
                    bool fenced = false;
                    if (p.win_ready && ti.phase == 0 && ti.window > waited_window) {
                        if (!flag_wait(p.win_ready + ti.window, p.win_ready_target, abort_flag, p.status, kWaitWindowReady, ti.window)) { ok = false; break; }
                        waited_window = ti.window;
                        fenced = true;
                    }
                    if (MODE == MODE_FWD && ti.phase == 1) {
                        if (!flag_wait(p.blk_done + (ti.m_blk - sched.m_first), sched.n_gu * 4 * NCTA, abort_flag, p.status, kWaitBlockDone, ti.m_blk - sched.m_first)) { ok = false; break; }
                        fenced = true;
                    }
                    if (fenced) fence_proxy_async_global();
                }
                for (int it = 0; it < ti.k_iters; ++it) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                    const uint32_t fb_local = full_bar(s);
                    const uint32_t fb = NCTA == 2 ? map_to_cta(fb_local, 0) : fb_local;
                    if (cta == 0) mbar_expect_tx(fb_local, NCTA * STAGE_BYTES);
                    const uint32_t a_dst = smem_base + s * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_BYTES;
                    const int bcol0 = ti.n_blk * BN + static_cast<int>(cta) * G::B_COLS;    // this CTA's B columns
                    if (MODE == MODE_NT) {
                        tma_tile<NCTA>(a_dst, &tmA, fb, it * BK, row0);
                        tma_tile<NCTA>(b_dst, &tmB, fb, it * BK, ti.group * p.b_rows_per_group + bcol0);
                    } else if (MODE == MODE_FWD && ti.phase == 1) {
                        tma_tile<NCTA>(a_dst, &tmA2, fb, it * BK, row0);
                        tma_tile<NCTA>(b_dst, &tmB3, fb, it * BK, ti.group * p.b3_rows_per_group + bcol0);
                    } else if (MODE == MODE_SWIGLU || MODE == MODE_FWD) {
                        tma_tile<NCTA>(a_dst, &tmA, fb, it * BK, row0);
                        const int brow = ti.group * p.b_rows_per_group + ti.n_blk * 128;
                        if (NCTA == 2) {      // leader stages the gate columns, its peer the up columns
                            tma_tile<NCTA>(b_dst, cta == 0 ? &tmB : &tmB2, fb, it * BK, brow);
                        } else {
                            tma_tile<NCTA>(b_dst, &tmB, fb, it * BK, brow);
                            tma_tile<NCTA>(b_dst + G::B_BYTES / 2, &tmB2, fb, it * BK, brow);
                        }
                    } else if (MODE == MODE_NN) {
                        const bool second = it >= kh;
                        const int kk = (second ? it - kh : it) * BK;
                        const CUtensorMap* ta = second ? &tmA2 : &tmA;
                        const CUtensorMap* tb = second ? &tmB2 : &tmB;
                        tma_tile<NCTA>(a_dst, ta, fb, kk, row0);
                        const int brow = ti.group * p.b_rows_per_group + kk;
#pragma unroll
                        for (int c = 0; c < G::B_COLS / 64; ++c) tma_tile<NCTA>(b_dst + c * CHUNK_BYTES, tb, fb, bcol0 + 64 * c, brow);
                    } else {
                        const int krow = ti.k_row0 + it * BK;
#pragma unroll
                        for (int c = 0; c < 2; ++c) tma_tile<NCTA>(a_dst + c * CHUNK_BYTES, &tmA, fb, row0 + 64 * c, krow);
#pragma unroll
                        for (int c = 0; c < G::B_COLS / 64; ++c) tma_tile<NCTA>(b_dst + c * CHUNK_BYTES, &tmB, fb, bcol0 + 64 * c, krow);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && cta == 0) {
            constexpr uint32_t a_mn = MODE == MODE_WGRAD ? 1u : 0u;
            constexpr uint32_t b_mn = (MODE == MODE_NN || MODE == MODE_WGRAD) ? 1u : 0u;
            // instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128 per CTA, N = 256
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (a_mn << 15) | (b_mn << 16) |
                                       (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(G::TILE_M >> 4) << 24);
            constexpr uint32_t a_step = a_mn ? (2048u >> 4) : (32u >> 4);   // descriptor advance per 16 elements of K
            constexpr uint32_t b_step = b_mn ? (2048u >> 4) : (32u >> 4);
            constexpr uint16_t pair_mask = 0x3;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int local = 0;
            Tile next_ti = {};
            if (tile_id0 < sched.total) next_ti = sched.get(p, tile_id0);
            for (int t = tile_id0; ok && t < sched.total; t += tile_stride, ++local) {
                const Tile ti = next_ti;
                if (t + tile_stride < sched.total) next_ti = sched.get(p, t + tile_stride);
                const int acc = local & 1;
                const uint32_t acc_ph = (local >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int it = 0; it < ti.k_iters; ++it) {
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * STAGE_BYTES;
                    const uint32_t b_addr = a_addr + A_BYTES;
                    const uint64_t a_desc = a_mn ? make_smem_desc(a_addr, CHUNK_BYTES, 1024) : make_smem_desc(a_addr, 16, 1024);
                    const uint64_t b_desc = b_mn ? make_smem_desc(b_addr, CHUNK_BYTES, 1024) : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = a_desc + static_cast<uint64_t>(k * a_step);
                        const uint64_t bd = b_desc + static_cast<uint64_t>(k * b_step);
                        if (NCTA == 2) umma_bf16_pair(d_tmem, ad, bd, idesc, (it | k) != 0 ? 1u : 0u);
                        else umma_bf16(d_tmem, ad, bd, idesc, (it | k) != 0 ? 1u : 0u);
                    }
                    // frees the smem stage (in both CTAs) once these MMAs retire
                    if (NCTA == 2) umma_commit_pair(empty_bar(s), pair_mask);
                    else umma_commit(empty_bar(s));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                // accumulator complete -> epilogue warps (of both CTAs)
                if (NCTA == 2) umma_commit_pair(tfull_bar(acc), pair_mask);
                else umma_commit(tfull_bar(acc));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5 of every CTA)
        const int quarter = warp & 3;                   // TMEM lanes [32q, 32q+32) belong to warps with id % 4 == q
        const int row_in_cta = quarter * 32 + lane;
        int local = 0;
        bool ok = true;
        for (int t = tile_id0; ok && t < sched.total; t += tile_stride, ++local) {
            const Tile ti = sched.get(p, t);
            const int acc = local & 1;
            const uint32_t acc_ph = (local >> 1) & 1u;
            if (!mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, MOKB_ST_PIPELINE_TIMEOUT)) { ok = false; break; }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            const bool empty_k = ti.k_iters == 0;
            const int row_in_tile = static_cast<int>(cta) * 128 + row_in_cta;
            if (MODE == MODE_SWIGLU || (MODE == MODE_FWD && ti.phase == 0)) {
                const size_t row = static_cast<size_t>(ti.m_blk) * G::TILE_M + row_in_tile;
                const size_t off = row * p.ldd + static_cast<size_t>(ti.n_blk) * 128;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_addr + c * 32, g);
                    tmem_ld_32x32(t_addr + 128 + c * 32, u);
                    tmem_ld_wait();
                    uint32_t h[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float gf = bf16_round(__uint_as_float(g[i]));
                        float uf = bf16_round(__uint_as_float(u[i]));
                        g[i] = __float_as_uint(gf);
                        u[i] = __float_as_uint(uf);
                        if (p.has_limit) {
                            gf = fminf(gf, p.limit);
                            uf = fminf(fmaxf(uf, -p.limit), p.limit);
                        }
                        h[i] = __float_as_uint(gf / (1.0f + __expf(-gf)) * uf);
                    }
                    store_row32(p.D + off + c * 32, g, p.wide_stores);
                    store_row32(p.D2 + off + c * 32, u, p.wide_stores);
                    store_row32(p.D3 + off + c * 32, h, p.wide_stores);
                }
            } else {
                const int tile_row = ti.m_blk * G::TILE_M + row_in_tile;
                bool row_ok = true;
                size_t row;
                if (MODE == MODE_WGRAD) {
                    row_ok = tile_row < p.M;
                    row = static_cast<size_t>(ti.group) * p.M + tile_row;
                } else {
                    row = static_cast<size_t>(tile_row);
                }
                __nv_bfloat16* const base = MODE == MODE_FWD ? p.D4 : p.D;
                const size_t ld_out = MODE == MODE_FWD ? p.ldd4 : p.ldd;
                __nv_bfloat16* dst = base + row * ld_out + static_cast<size_t>(ti.n_blk) * BN;
                if (base == nullptr) row_ok = false;          // pushed only
                __nv_bfloat16* pdst = nullptr;                // this row's place in its home rank's buffer
                if ((MODE == MODE_NT || MODE == MODE_NN || MODE == MODE_FWD) && p.push) {
                    const int pr = p.push_rank[tile_row];
                    if (pr >= 0 && pr < p.push_ranks &&
                        index_ok(IndexGuard{p.push_limit, p.status}, p.push_idx[tile_row], kBadIndexGemmPush, tile_row)) {
                        const size_t slot = static_cast<size_t>(p.push_idx[tile_row]);
                        pdst = static_cast<__nv_bfloat16*>(p.push_dst.p[pr]) + slot * ld_out + static_cast<size_t>(ti.n_blk) * BN;
                        if (p.push_values && ti.n_blk == 0) static_cast<float*>(p.push_val.p[pr])[slot] = p.push_values[tile_row];
                    }
                }
                const int cols_left = (MODE == MODE_FWD ? p.N2 : p.N) - ti.n_blk * BN;
                const int nchunks = min(BN / 32, (cols_left + 31) / 32);
                // one 32-column chunk from registers: (optionally add the stored gradient,) round to bf16, store locally
                // and / or at home
                auto put = [&](uint32_t (&r)[32], int c) {
                    if (MODE == MODE_WGRAD && p.accumulate && row_ok) {
                        const uint4* old = reinterpret_cast<const uint4*>(dst + c * 32);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 o = old[q];
                            const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = unpack_bf16(ow[j]);
                                r[8 * q + 2 * j] = __float_as_uint(__uint_as_float(r[8 * q + 2 * j]) + f.x);
                                r[8 * q + 2 * j + 1] = __float_as_uint(__uint_as_float(r[8 * q + 2 * j + 1]) + f.y);
                            }
                        }
                    }
                    if (row_ok) store_row32(dst + c * 32, r, p.wide_stores);
                    if (pdst) store_row32(pdst + c * 32, r, p.push_wide);
                };
                if (empty_k) {
                    if (!(MODE == MODE_WGRAD && p.accumulate)) {      // accumulate: nothing to add, leave the stored gradient
                        uint32_t z[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) z[i] = 0u;
#pragma unroll 1
                        for (int c = 0; c < nchunks; ++c) put(z, c);
                    }
                } else if ((MODE == MODE_WGRAD && p.accumulate) || (nchunks & 1) || !p.line_stores) {
                    // register path: a lane stores its own row, 32 bytes at a time.  Two register sets: the tensor-memory
                    // load of the next chunk is in flight while this one is stored (whole warp, also for unstored rows)
                    uint32_t ra[32], rb[32];
                    tmem_ld_32x32(t_addr, ra);
                    tmem_ld_wait_for(ra);
#pragma unroll 1
                    for (int c = 0; c < nchunks; c += 2) {
                        const bool has_b = c + 1 < nchunks, has_next = c + 2 < nchunks;
                        if (has_b) tmem_ld_32x32(t_addr + (c + 1) * 32, rb);
                        put(ra, c);
                        if (has_b) {
                            tmem_ld_wait_for(rb);
                            if (has_next) tmem_ld_32x32(t_addr + (c + 2) * 32, ra);
                            put(rb, c + 1);
                            if (has_next) tmem_ld_wait_for(ra);
                        }
                    }
                } else {
                    // line path: 64 columns (128 bytes) of the warp's 32 rows are transposed through shared memory, so
                    // that eight lanes store one whole 128-byte line of a row and a store instruction touches 4 lines
                    // instead of 32 sectors of 32 different lines -- what the L2 and, for rows that go to a peer, the
                    // NVLink packets are made for.
                    const uint32_t stage = bars + 256u + static_cast<uint32_t>(warp - 2) * 4096u;
                    const int sub = lane >> 3, unit = lane & 7;
                    // lane 0's row of the local output (rows of a warp are consecutive) and this lane's own row at home
                    __nv_bfloat16* const warp_dst = base ? dst - static_cast<size_t>(lane) * ld_out : nullptr;
                    const int warp_row0 = tile_row - lane;
                    const unsigned long long own_home = reinterpret_cast<unsigned long long>(pdst);
                    const int npairs = nchunks >> 1;
#pragma unroll 1
                    for (int cp = 0; cp < npairs; ++cp) {
                        uint32_t w[32];           // this lane's row, 64 columns as bf16 pairs
                        {
                            uint32_t ra[32], rb[32];
                            tmem_ld_32x32(t_addr + (2 * cp) * 32, ra);
                            tmem_ld_32x32(t_addr + (2 * cp + 1) * 32, rb);
                            tmem_ld_wait_for(ra);
                            tmem_ld_wait_for(rb);
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                w[i] = pack_bf16(__uint_as_float(ra[2 * i]), __uint_as_float(ra[2 * i + 1]));
                                w[16 + i] = pack_bf16(__uint_as_float(rb[2 * i]), __uint_as_float(rb[2 * i + 1]));
                            }
                        }
                        __syncwarp();             // the previous pair has been read out of the buffer
#pragma unroll
                        for (int u = 0; u < 8; ++u)      // row `lane`, 16-byte unit u at position u ^ (lane & 7): conflict-free both ways
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128u + static_cast<uint32_t>((u ^ (lane & 7)) << 4)),
                                         "r"(w[4 * u]), "r"(w[4 * u + 1]), "r"(w[4 * u + 2]), "r"(w[4 * u + 3]) : "memory");
                        __syncwarp();
                        const int col = cp * 64 + unit * 8;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = 4 * i + sub;
                            uint32_t v0, v1, v2, v3;
                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                         : "r"(stage + rr * 128u + static_cast<uint32_t>((unit ^ (rr & 7)) << 4)) : "memory");
                            if (warp_dst && (MODE != MODE_WGRAD || warp_row0 + rr < p.M))
                                st_global_v4(warp_dst + static_cast<size_t>(rr) * ld_out + col, v0, v1, v2, v3);
                            if ((MODE == MODE_NT || MODE == MODE_NN || MODE == MODE_FWD) && p.push) {
                                __nv_bfloat16* home = reinterpret_cast<__nv_bfloat16*>(__shfl_sync(0xffffffffu, own_home, rr));
                                if (home) st_global_v4(home + col, v0, v1, v2, v3);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (NCTA == 2) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
                else mbar_arrive(tempty_bar(acc));
                if (MODE == MODE_FWD) {
                    // this warp's rows of the tile are stored: count it for whoever reads them next
                    int32_t* counter = ti.phase == 0 ? p.blk_done + (ti.m_blk - sched.m_first) : (p.win_done ? p.win_done + ti.window : nullptr);
                    if (counter) red_release_gpu_add(counter, 1);
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: give copies still in flight time to land before the CTA's smem is released
        const unsigned long long t0 = clock64();
        while (clock64() - t0 < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (NCTA == 2) cluster_sync_all();     // the peer may still read this CTA's smem or signal its barriers until here
    if (warp == 1) {
        tc_fence_after();
        if (NCTA == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int MODE, int NCTA>
int launch(const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2, const CUtensorMap& b2, const CUtensorMap& b3,
           const KParams& p, int tiles_upper_bound, cudaStream_t stream) {
    const size_t smem = Geo<NCTA>::SMEM_BYTES - (p.line_stores ? 0 : 4 * 4096);
    MOKB_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<MODE, NCTA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Geo<NCTA>::SMEM_BYTES));
    int units = sm_count() / NCTA;                       // CTAs, or CTA pairs
    // a launch that waits for another kernel's rows leaves one pair of SMs to that kernel: whatever else shares the
    // GPU, the rows it waits for can always be produced
    if (p.win_ready && units > 2) units -= 2 / NCTA;
    if (tiles_upper_bound < units) units = tiles_upper_bound;
    if (units < 1) return MOKB_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(units * NCTA));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = NCTA;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MOKB_CUDA(cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<MODE, NCTA>, a, b, a2, b2, b3, p));
    note_launch();
    return MOKB_OK;
}

// MOKB_GEMM_CTAS=1 selects the single-CTA tile (for comparison); the default is the CTA pair.
int ctas_per_tile() {
    static int v = 0;
    if (v == 0) {
        const char* e = getenv("MOKB_GEMM_CTAS");
        v = (e && e[0] == '1') ? 1 : 2;
    }
    return v;
}

template <int MODE>
int dispatch_launch(int ncta, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& a2, const CUtensorMap& b2,
                    const KParams& p, int tiles, cudaStream_t stream) {
    return ncta == 2 ? launch<MODE, 2>(a, b, a2, b2, b, p, tiles, stream) : launch<MODE, 1>(a, b, a2, b2, b, p, tiles, stream);
}

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" int mokb_grouped_gemm_bf16(const mokb_gemm_args* g, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_REQUIRE(g != nullptr, "grouped_gemm: null args");
    MOKB_REQUIRE(g->mode >= 0 && g->mode <= 4, "grouped_gemm: unknown mode %d", g->mode);
    static const char* const kTags[5] = {"gemm_bf16_nt", "gemm_bf16_gate_up_swiglu", "gemm_bf16_nn", "gemm_bf16_wgrad", "gemm_bf16_fwd_routed"};
    TraceScope trace(stream, kTags[g->mode], g->row_begin);
    MOKB_REQUIRE(g->A && g->B && g->status, "grouped_gemm: null pointer");
    MOKB_REQUIRE(g->D || (g->push_ptrs_host && g->mode != MODE_FWD), "grouped_gemm: D may only be left out when the result is pushed to peers");
    MOKB_REQUIRE(g->G >= 1, "grouped_gemm: G must be >= 1");
    MOKB_REQUIRE(g->rows_static >= 0 && g->rows_static % 128 == 0, "grouped_gemm: rows must be a multiple of 128");
    // row tiles of 256 need row counts in multiples of 256 (true for every tensor of the layer)
    const int ncta = (g->mode == MODE_FWD || (ctas_per_tile() == 2 && g->rows_static % 256 == 0)) ? 2 : 1;
    MOKB_REQUIRE(g->mode != MODE_FWD || g->rows_static % 256 == 0, "grouped_gemm FWD: rows must be a multiple of 256");
    const int TM = 128 * ncta;
    const uint32_t b_box = static_cast<uint32_t>(BN / ncta);
    KParams p;
    memset(&p, 0, sizeof(p));
    p.rows_cap = g->rows_static;
    p.row_begin = g->row_begin;
    p.row_end = g->row_end > 0 ? g->row_end : g->rows_static;
    MOKB_REQUIRE(p.row_begin >= 0 && p.row_begin % 256 == 0 && p.row_end % (128 * ncta) == 0 && p.row_begin <= p.row_end && p.row_end <= g->rows_static,
                 "grouped_gemm: bad row window [%d, %d) of %d", g->row_begin, g->row_end, g->rows_static);
    p.num_rows = g->num_rows;
    p.group_of_block = g->group_of_block;
    p.group_offsets = g->group_offsets;
    p.group_k_end = g->mode == MODE_WGRAD ? g->group_k_end : nullptr;
    p.G = g->G; p.M = g->M; p.N = g->N; p.K = g->K;
    p.D = static_cast<__nv_bfloat16*>(g->D);
    p.D2 = static_cast<__nv_bfloat16*>(g->D2);
    p.D3 = static_cast<__nv_bfloat16*>(g->D3);
    p.ldd = g->ldd;
    p.wide_stores = g->ldd % 16 == 0 && ((reinterpret_cast<uintptr_t>(g->D) | reinterpret_cast<uintptr_t>(g->D2) |
                                          reinterpret_cast<uintptr_t>(g->D3)) & 31) == 0;
    p.accumulate = g->accumulate;
    p.has_limit = g->has_swiglu_limit;
    p.limit = g->swiglu_limit;
    p.status = g->status;
    p.dual = 0;
    { const char* e = getenv("MOKB_LINE_STORES"); p.line_stores = e ? atoi(e) : 1; }
    if (g->push_ptrs_host) {
        MOKB_REQUIRE(g->mode == MODE_NT || g->mode == MODE_NN || g->mode == MODE_FWD, "grouped_gemm: push is for modes 0, 2 and 4");
        MOKB_REQUIRE(g->push_ep_size >= 1 && g->push_ep_size <= MOKB_MAX_EP && g->push_rank && g->push_idx, "grouped_gemm: push needs ranks and indices");
        MOKB_REQUIRE((g->push_values == nullptr) == (g->push_value_ptrs_host == nullptr), "grouped_gemm: push_values and push_value_ptrs_host go together");
        const int ld_out = g->mode == MODE_FWD ? g->ldd4 : g->ldd;
        MOKB_REQUIRE(g->push_index_limit >= 0 && g->push_index_limit <= INT32_MAX, "grouped_gemm: push_index_limit must fit 31 bits");
        p.push_limit = static_cast<int>(g->push_index_limit);
        p.push = 1; p.push_ranks = g->push_ep_size; p.push_rank = g->push_rank; p.push_idx = g->push_idx; p.push_values = g->push_values;
        p.push_wide = ld_out % 16 == 0;
        for (int r = 0; r < kPeerMax; ++r) p.push_dst.p[r] = p.push_val.p[r] = nullptr;
        for (int r = 0; r < g->push_ep_size; ++r) {
            MOKB_REQUIRE(g->push_ptrs_host[r] != 0 && (g->push_ptrs_host[r] & 15) == 0, "grouped_gemm: push pointer of rank %d is null or not 16-byte aligned", r);
            p.push_dst.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(g->push_ptrs_host[r]));
            if ((g->push_ptrs_host[r] & 31) != 0) p.push_wide = 0;
            if (g->push_value_ptrs_host) {
                MOKB_REQUIRE(g->push_value_ptrs_host[r] != 0, "grouped_gemm: push value pointer of rank %d is null", r);
                p.push_val.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(g->push_value_ptrs_host[r]));
            }
        }
    }
    if (g->mode != MODE_WGRAD) {
        MOKB_REQUIRE(g->window_rows >= 0 && g->window_rows % 256 == 0, "grouped_gemm: window_rows must be a multiple of 256");
        MOKB_REQUIRE(g->win_ready == nullptr || (g->window_rows > 0 && g->win_ready_target > 0), "grouped_gemm: win_ready needs window_rows and a target");
        p.window_rows = g->window_rows;
        p.win_ready = g->win_ready;
        p.win_ready_target = g->win_ready_target;
    }
    MOKB_REQUIRE(g->ldd % 8 == 0 && g->lda % 8 == 0 && g->ldb % 8 == 0, "grouped_gemm: leading dimensions must be multiples of 8");
    MOKB_REQUIRE((reinterpret_cast<uintptr_t>(g->D) & 15) == 0, "grouped_gemm: D not 16-byte aligned");
    if (g->rows_static == 0) return MOKB_OK;
    const uint64_t rows = static_cast<uint64_t>(g->rows_static);
    const int m_tiles = (p.row_end - p.row_begin + TM - 1) / TM;
    CUtensorMap ta, tb, ta2, tb2;
    switch (g->mode) {
    case MODE_NT: {
        MOKB_REQUIRE(g->K > 0 && g->K % BK == 0 && g->N > 0 && g->N % BN == 0, "grouped_gemm NT: K %% 64 and N %% 256 must be 0");
        MOKB_TRY(make_tmap_2d(&ta, g->A, 2, g->K, rows, 2ull * g->lda, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb, g->B, 2, g->K, static_cast<uint64_t>(g->G) * g->N, 2ull * g->ldb, 64, b_box));
        p.b_rows_per_group = g->N;
        ta2 = ta; tb2 = tb;
        return dispatch_launch<MODE_NT>(ncta, ta, tb, ta2, tb2, p, m_tiles * (g->N / BN), stream);
    }
    case MODE_SWIGLU: {
        MOKB_REQUIRE(g->K > 0 && g->K % BK == 0 && g->N > 0 && g->N % 128 == 0, "grouped_gemm SWIGLU: K %% 64 and N %% 128 must be 0");
        MOKB_REQUIRE(g->B2 && g->D2 && g->D3, "grouped_gemm SWIGLU: B2, D2, D3 required");
        MOKB_TRY(make_tmap_2d(&ta, g->A, 2, g->K, rows, 2ull * g->lda, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb, g->B, 2, g->K, static_cast<uint64_t>(g->G) * g->N, 2ull * g->ldb, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb2, g->B2, 2, g->K, static_cast<uint64_t>(g->G) * g->N, 2ull * g->ldb, 64, 128));
        p.b_rows_per_group = g->N;
        ta2 = ta;
        return dispatch_launch<MODE_SWIGLU>(ncta, ta, tb, ta2, tb2, p, m_tiles * (g->N / 128), stream);
    }
    case MODE_NN: {
        MOKB_REQUIRE(g->K > 0 && g->K % BK == 0 && g->N > 0 && g->N % 64 == 0, "grouped_gemm NN: K %% 64 and N %% 64 must be 0");
        MOKB_REQUIRE((g->A2 == nullptr) == (g->B2 == nullptr), "grouped_gemm NN: A2 and B2 go together");
        MOKB_TRY(make_tmap_2d(&ta, g->A, 2, g->K, rows, 2ull * g->lda, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb, g->B, 2, g->N, static_cast<uint64_t>(g->G) * g->K, 2ull * g->ldb, 64, 64));
        ta2 = ta; tb2 = tb;
        if (g->A2) {
            MOKB_TRY(make_tmap_2d(&ta2, g->A2, 2, g->K, rows, 2ull * g->lda, 64, 128));
            MOKB_TRY(make_tmap_2d(&tb2, g->B2, 2, g->N, static_cast<uint64_t>(g->G) * g->K, 2ull * g->ldb, 64, 64));
            p.dual = 1;
        }
        p.b_rows_per_group = g->K;
        return dispatch_launch<MODE_NN>(ncta, ta, tb, ta2, tb2, p, m_tiles * ((g->N + BN - 1) / BN), stream);
    }
    case MODE_FWD: {
        MOKB_REQUIRE(g->K > 0 && g->K % BK == 0 && g->N > 0 && g->N % 128 == 0, "grouped_gemm FWD: K %% 64 and N %% 128 must be 0");
        MOKB_REQUIRE(g->B2 && g->D2 && g->D3 && g->blk_done, "grouped_gemm FWD: B2, D2, D3 and blk_done required");
        MOKB_REQUIRE(g->N2 >= 0 && g->N2 % BN == 0, "grouped_gemm FWD: N2 must be a multiple of 256");
        MOKB_TRY(make_tmap_2d(&ta, g->A, 2, g->K, rows, 2ull * g->lda, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb, g->B, 2, g->K, static_cast<uint64_t>(g->G) * g->N, 2ull * g->ldb, 64, 128));
        MOKB_TRY(make_tmap_2d(&tb2, g->B2, 2, g->K, static_cast<uint64_t>(g->G) * g->N, 2ull * g->ldb, 64, 128));
        p.b_rows_per_group = g->N;
        ta2 = ta;
        CUtensorMap tb3 = tb;
        if (g->N2 > 0) {
            // the down projection reads the hidden rows this launch writes: A2 = D3 [rows, N], contraction over N
            MOKB_REQUIRE(g->B3 && (g->D4 || g->push_ptrs_host) && g->ldd4 > 0 && g->ldd4 % 8 == 0 && g->ldb3 % 8 == 0,
                         "grouped_gemm FWD: B3, D4 (or push pointers) and their leading dimensions required");
            MOKB_REQUIRE(g->N % BK == 0, "grouped_gemm FWD: N must be a multiple of 64 for the down projection");
            MOKB_REQUIRE((reinterpret_cast<uintptr_t>(g->D4) & 15) == 0, "grouped_gemm FWD: D4 not 16-byte aligned");
            MOKB_TRY(make_tmap_2d(&ta2, g->D3, 2, g->N, rows, 2ull * g->ldd, 64, 128));
            MOKB_TRY(make_tmap_2d(&tb3, g->B3, 2, g->N, static_cast<uint64_t>(g->G) * g->N2, 2ull * g->ldb3, 64, 128));
            p.N2 = g->N2; p.K2 = g->N; p.b3_rows_per_group = g->N2;
            p.D4 = static_cast<__nv_bfloat16*>(g->D4); p.ldd4 = g->ldd4;
            p.wide_stores = p.wide_stores && g->ldd4 % 16 == 0 && (reinterpret_cast<uintptr_t>(g->D4) & 31) == 0;
        }
        p.blk_done = g->blk_done;
        p.win_done = g->win_done;
        return launch<MODE_FWD, 2>(ta, tb, ta2, tb2, tb3, p, m_tiles * (g->N / 128 + g->N2 / BN), stream);
    }
    default: {
        MOKB_REQUIRE(g->M > 0 && g->M % 128 == 0 && g->N > 0 && g->N % 64 == 0, "grouped_gemm WGRAD: M %% 128 and N %% 64 must be 0");
        MOKB_REQUIRE(g->group_offsets != nullptr, "grouped_gemm WGRAD: group_offsets required");
        MOKB_TRY(make_tmap_2d(&ta, g->A, 2, g->M, rows, 2ull * g->lda, 64, 64));
        MOKB_TRY(make_tmap_2d(&tb, g->B, 2, g->N, rows, 2ull * g->ldb, 64, 64));
        ta2 = ta; tb2 = tb;
        const int wg_ncta = ctas_per_tile();     // the weight-gradient tile is over M and N, not over rows
        const int tm = 128 * wg_ncta;
        return dispatch_launch<MODE_WGRAD>(wg_ncta, ta, tb, ta2, tb2, p, g->G * ((g->M + tm - 1) / tm) * ((g->N + BN - 1) / BN), stream);
    }
    }
}
