// MXFP8 codec kernels: bf16 -> E4M3 with one E8M0 scale per 32 elements, along rows
// ("normal") and/or along columns ("transposed": the quantisation of x^T), scales laid out
// in the 32 x 16-byte tiles that tcgen05 block-scaled MMA consumes.
//   quantize_kernel         plain quantiser            (reference: csrc/mxfp8.cuh:188-278)
//   (SwiGLU forward + quantise is the epilogue of the MXFP8 gate/up GEMM, gemm_mxfp8.cu)
//   swiglu_bwd_quant_kernel de-quantise saved gate/up, SwiGLU backward, router-gradient partials,
//                           quantise d_gate / d_up      (reference: swiglu.cuh:209-566)
// One 128 x 128 tile per CTA, staged in shared memory as packed bf16 pairs with an odd word pitch,
// so that the row-wise pass (a thread owns 32 columns of one row) and the column-wise pass (a
// thread owns 32 rows of two adjacent columns) both read it without bank conflicts.  The kernels
// are bound by HBM, but only if the per-element instruction count stays small: everything works on
// bf16 pairs (packed abs/max for the block maximum, one conversion instruction per two outputs)
// and global memory is touched 32 bytes per thread per instruction.
#include <cuda_fp8.h>

#include "common.cuh"
#include "mxfp8_codec.cuh"

namespace mokb {
namespace {

constexpr int TILE = 128;
constexpr int WPITCH = TILE / 2 + 1;          // 32-bit words per smem row (65: odd)
constexpr int TILE_WORDS = TILE * WPITCH;

// Row-wise quantisation of a staged tile into q [rows, cols] (+ scales): item = (row, block of 32 columns);
// consecutive lanes take consecutive rows (conflict-free with the odd pitch).
__device__ __forceinline__ void quantize_tile_rows(const uint32_t* tile, uint8_t* q, uint8_t* sc, int64_t row_base,
                                                   int64_t r0, int64_t c0, int64_t cols) {
    for (int item = threadIdx.x; item < TILE * 4; item += blockDim.x) {
        const int r = item & 127, kb = item >> 7;
        uint32_t w[16];
        uint32_t m = 0u;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            w[i] = tile[r * WPITCH + kb * 16 + i];
            m = absmax2(m, w[i]);
        }
        float inv;
        const uint32_t byte = scale_byte(fmaxf(bf16_lo(m), bf16_hi(m)), &inv);
        uint32_t out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            out[i] = e4m3x4(bf16_lo(w[2 * i]) * inv, bf16_hi(w[2 * i]) * inv, bf16_lo(w[2 * i + 1]) * inv, bf16_hi(w[2 * i + 1]) * inv);
        st_global_32B(q + (row_base + r0 + r) * cols + c0 + kb * 32, out);
        sc[scale_offset(row_base + r0 + r, (c0 >> 5) + kb, cols >> 7)] = static_cast<uint8_t>(byte);
    }
}

// Column-wise quantisation into qt [cols, rows] (+ scales): item = (pair of adjacent columns, block of 32 rows);
// consecutive lanes take consecutive column pairs.
__device__ __forceinline__ void quantize_tile_cols(const uint32_t* tile, uint8_t* qt, uint8_t* sct, int64_t col_base,
                                                   int64_t r0, int64_t c0, int64_t rows) {
    for (int item = threadIdx.x; item < (TILE / 2) * 4; item += blockDim.x) {
        const int cp = item & 63, kb = item >> 6;
        uint32_t w[32];
        uint32_t m = 0u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            w[i] = tile[(kb * 32 + i) * WPITCH + cp];
            m = absmax2(m, w[i]);
        }
        float inv_a, inv_b;
        const uint32_t byte_a = scale_byte(bf16_lo(m), &inv_a);
        const uint32_t byte_b = scale_byte(bf16_hi(m), &inv_b);
        uint32_t out[8];
        const int64_t col = col_base + c0 + 2 * cp;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            out[i] = e4m3x4(bf16_lo(w[4 * i]) * inv_a, bf16_lo(w[4 * i + 1]) * inv_a, bf16_lo(w[4 * i + 2]) * inv_a, bf16_lo(w[4 * i + 3]) * inv_a);
        st_global_32B(qt + col * rows + r0 + kb * 32, out);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            out[i] = e4m3x4(bf16_hi(w[4 * i]) * inv_b, bf16_hi(w[4 * i + 1]) * inv_b, bf16_hi(w[4 * i + 2]) * inv_b, bf16_hi(w[4 * i + 3]) * inv_b);
        st_global_32B(qt + (col + 1) * rows + r0 + kb * 32, out);
        sct[scale_offset(col, (r0 >> 5) + kb, rows >> 7)] = static_cast<uint8_t>(byte_a);
        sct[scale_offset(col + 1, (r0 >> 5) + kb, rows >> 7)] = static_cast<uint8_t>(byte_b);
    }
}

// 128 x 128 bf16 from global memory (row stride ld elements) into a staged tile, 32 bytes per thread per load
__device__ __forceinline__ void load_tile_bf16(uint32_t* tile, const __nv_bfloat16* src, int64_t ld) {
    // 1024 chunks of 32 bytes over 256 threads: all four loads are issued before the first store
    uint32_t val[4][8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + 256 * k;
        ld_global_32B(src + static_cast<int64_t>(i >> 3) * ld + (i & 7) * 16, val[k]);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + 256 * k;
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[(i >> 3) * WPITCH + (i & 7) * 8 + j] = val[k][j];
    }
}

// Rows [begin, min(end, *num_rows)); the grid's y index counts 128-row tiles from `begin`.  Row numbers are those of the
// caller's row space (the schedule's, for the layer): a buffer that holds only rows [first, first + M) of it is passed
// with its pointers moved back by `first` rows, so begin/end may exceed the buffer's own row count M.
struct RowWindow {
    const int32_t* num_rows;
    int begin, end;
};
__device__ __forceinline__ bool tile_in_window(const RowWindow& w, int64_t* r0) {
    *r0 = static_cast<int64_t>(blockIdx.y) * TILE + w.begin;
    const int live = w.num_rows ? min(max(*w.num_rows, 0), w.end) : w.end;
    return *r0 < live;
}

// 256 threads per block; the blocks of the launch walk the 128 x 128 tiles of the window (column tiles fastest).
__global__ void __launch_bounds__(256) quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t E, int64_t M, int64_t N,
                                                       RowWindow win,
                                                       uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                                       uint8_t* __restrict__ qt, uint8_t* __restrict__ sct, int32_t* done_counter) {
    __shared__ uint32_t tile[TILE_WORDS];
    const int live = win.num_rows ? min(max(*win.num_rows, 0), win.end) : win.end;
    const int64_t row_tiles = live > win.begin ? (live - win.begin + TILE - 1) / TILE : 0;
    const int64_t col_tiles = N / TILE;
    const int64_t ntiles = E * row_tiles * col_tiles;
    for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int64_t e = t / (row_tiles * col_tiles);
        const int64_t rem = t - e * row_tiles * col_tiles;
        const int64_t rt = rem / col_tiles;
        const int64_t c0 = (rem - rt * col_tiles) * TILE;
        const int64_t r0 = win.begin + rt * TILE;
        load_tile_bf16(tile, x + (e * M + r0) * N + c0, N);
        __syncthreads();
        if (q) quantize_tile_rows(tile, q, sc, e * M, r0, c0, N);
        if (qt) quantize_tile_cols(tile, qt, sct, e * N, r0, c0, M);
        __syncthreads();          // the tile is free for the next load
    }
    if (done_counter) {      // one arrival per block of the launch (also those without tiles): the window is quantised
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            red_release_gpu_add(done_counter, 1);
        }
    }
}

// Column-wise ("transposed") quantisation only, for tensors whose row-wise form already exists (the dispatch kernel
// writes it as the rows arrive): qt [N, M] + scales from x [M, N].  No shared memory and at most 64 registers, so that
// two blocks of 128 threads fit on an SM beside any of the GEMM kernels (the MXFP8 GEMM leaves less than 8 KB of
// shared memory and 4096 registers per SM quarter) and the pass runs under the GEMM instead of after it.  A lane owns
// a pair of adjacent columns over a block of 32 rows: its 32 loads are independent, and a warp's load of one row is
// one 128-byte line.  Same arithmetic as quantize_tile_cols.
constexpr int CTILE_COLS = 64;
__global__ void __maxnreg__(64) quantize_cols_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t N, RowWindow win,
                                                     uint8_t* __restrict__ qt, uint8_t* __restrict__ sct) {
    const int live = win.num_rows ? min(max(*win.num_rows, 0), win.end) : win.end;
    const int64_t row_tiles = live > win.begin ? (live - win.begin + TILE - 1) / TILE : 0;
    const int64_t col_tiles = N / CTILE_COLS;
    const int64_t ntiles = row_tiles * col_tiles;
    const int cp = threadIdx.x & 31, kb = threadIdx.x >> 5;      // a pair of adjacent columns, a block of 32 rows
    for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int64_t rt = t / col_tiles;
        const int64_t c0 = (t - rt * col_tiles) * CTILE_COLS;
        const int64_t r0 = win.begin + rt * TILE + kb * 32;
        const int64_t col = c0 + 2 * cp;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(x + r0 * N + col);
        const int64_t pitch = N / 2;                             // 32-bit words per row
        // pass 1: the block maximum of both columns, eight independent loads at a time; pass 2 reads the rows again
        // (cache hits) four at a time.  Keeping the 32 values (and the 32 row addresses) in registers across the
        // conversion would take about 170 registers; this way the kernel stays within 64.
        uint32_t m = 0u;
        const uint32_t* p1 = src;
#pragma unroll 1
        for (int g = 0; g < 4; ++g) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = __ldg(p1 + i * pitch);
#pragma unroll
            for (int i = 0; i < 8; ++i) m = absmax2(m, w[i]);
            p1 += 8 * pitch;
        }
        float inv_a, inv_b;
        const uint32_t byte_a = scale_byte(bf16_lo(m), &inv_a);
        const uint32_t byte_b = scale_byte(bf16_hi(m), &inv_b);
        uint32_t out_a[8], out_b[8];
        const uint32_t* p2 = src;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)       // (volatile: must stay a second load, not a reuse of pass 1's registers)
                asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(w[j]) : "l"(p2 + j * pitch));
            p2 += 4 * pitch;
            out_a[i] = e4m3x4(bf16_lo(w[0]) * inv_a, bf16_lo(w[1]) * inv_a, bf16_lo(w[2]) * inv_a, bf16_lo(w[3]) * inv_a);
            out_b[i] = e4m3x4(bf16_hi(w[0]) * inv_b, bf16_hi(w[1]) * inv_b, bf16_hi(w[2]) * inv_b, bf16_hi(w[3]) * inv_b);
        }
        st_global_32B(qt + col * M + r0, out_a);
        st_global_32B(qt + (col + 1) * M + r0, out_b);
        sct[scale_offset(col, r0 >> 5, M >> 7)] = static_cast<uint8_t>(byte_a);
        sct[scale_offset(col + 1, r0 >> 5, M >> 7)] = static_cast<uint8_t>(byte_b);
    }
}

struct Clamp {
    int on;
    float limit;
};


// two E4M3 bytes (the low 16 bits of v) -> two floats
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t v) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v & 0xffffu), __NV_E4M3);
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Row-wise quantisation of one whole 32-element block: 16 packed words in shared memory.
__device__ __forceinline__ void quantize_block_smem(const uint32_t* src, uint8_t* q_dst, uint8_t* sc_dst) {
    uint32_t w[16];
    uint32_t m = 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        w[j] = src[j];
        m = absmax2(m, w[j]);
    }
    float inv;
    const uint32_t byte = scale_byte(fmaxf(bf16_lo(m), bf16_hi(m)), &inv);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        out[j] = e4m3x4(bf16_lo(w[2 * j]) * inv, bf16_hi(w[2 * j]) * inv, bf16_lo(w[2 * j + 1]) * inv, bf16_hi(w[2 * j + 1]) * inv);
    st_global_32B(q_dst, out);
    *sc_dst = static_cast<uint8_t>(byte);
}

// Saved gate/up (E4M3 + scales), d_hidden bf16 -> d_gate, d_up, their row-wise and column-wise quantisations,
// and the per-(row, 128-column block) router-gradient partial sum(d_hidden * silu(g) * u) / w.
// grid (I/128, window rows/128), 256 threads: two threads per row, 64 columns (two scale blocks) each, columns in
// ascending order.  d_gate / d_up are quantised row-wise from registers and staged (two tiles) for the column-wise pass.
__global__ void __launch_bounds__(256, 3) swiglu_bwd_quant_kernel(
    const uint8_t* __restrict__ gate_q, const uint8_t* __restrict__ gate_sc, const uint8_t* __restrict__ up_q,
    const uint8_t* __restrict__ up_sc, const __nv_bfloat16* __restrict__ d_hidden, int64_t rows_cap, int64_t I,
    RowWindow win, Clamp c, const float* __restrict__ row_scale,
    uint8_t* dg_q, uint8_t* dg_sc, uint8_t* dg_qt, uint8_t* dg_sct,
    uint8_t* du_q, uint8_t* du_sc, uint8_t* du_qt, uint8_t* du_sct, float* __restrict__ partials) {
    extern __shared__ uint32_t sm[];
    uint32_t *tdg = sm, *tdu = sm + TILE_WORDS;
    __shared__ float row_part[TILE][2];
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * TILE;
    int64_t r0;
    if (!tile_in_window(win, &r0)) return;
    const int r = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int64_t row = r0 + r;
    const float w = row_scale ? row_scale[row] : 1.0f;
    const float inv_w = w > 0.0f ? 1.0f / w : 0.0f;
    float partial = 0.0f;
#pragma unroll 1
    for (int kb = half * 2; kb < half * 2 + 2; ++kb) {
        const int64_t col = c0 + kb * 32;
        const size_t sc_off = scale_offset(row, col >> 5, I >> 7);
        const float gs = __uint_as_float(static_cast<uint32_t>(gate_sc[sc_off]) << 23);
        const float us = __uint_as_float(static_cast<uint32_t>(up_sc[sc_off]) << 23);
        uint32_t gv[8], uv[8], dh[16];
        ld_global_32B(gate_q + row * I + col, gv);
        ld_global_32B(up_q + row * I + col, uv);
        ld_global_32B(d_hidden + row * I + col, reinterpret_cast<uint32_t (&)[8]>(dh[0]));
        ld_global_32B(d_hidden + row * I + col + 16, reinterpret_cast<uint32_t (&)[8]>(dh[8]));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float2 gq = e4m3x2_to_float2(gv[i >> 1] >> ((i & 1) * 16));
            const float2 uq = e4m3x2_to_float2(uv[i >> 1] >> ((i & 1) * 16));
            const float gg[2] = {gq.x * gs, gq.y * gs}, uu[2] = {uq.x * us, uq.y * us};
            const float dhv[2] = {bf16_lo(dh[i]), bf16_hi(dh[i])};
            float dg[2], du[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float g = gg[j], u = uu[j];
                bool g_ok = true, u_ok = true;
                if (c.on) {
                    g_ok = g <= c.limit;
                    u_ok = (u >= -c.limit) && (u <= c.limit);
                    g = fminf(g, c.limit);
                    u = fminf(fmaxf(u, -c.limit), c.limit);
                }
                const float sig = 1.0f / (1.0f + __expf(-g));
                const float silu = g * sig;
                const float dsilu = (1.0f - silu) * sig + silu;
                dg[j] = g_ok ? dsilu * u * dhv[j] : 0.0f;
                du[j] = u_ok ? silu * dhv[j] : 0.0f;
                partial += dhv[j] * inv_w * (silu * u);
            }
            tdg[r * WPITCH + kb * 16 + i] = pack2(dg[0], dg[1]);
            tdu[r * WPITCH + kb * 16 + i] = pack2(du[0], du[1]);
        }
        // row-wise pass on the words this thread has just staged (its own: no barrier needed)
        quantize_block_smem(tdg + r * WPITCH + kb * 16, dg_q + row * I + col, dg_sc + sc_off);
        quantize_block_smem(tdu + r * WPITCH + kb * 16, du_q + row * I + col, du_sc + sc_off);
    }
    row_part[r][half] = partial;
    __syncthreads();
    if (partials && half == 0) partials[row * (I >> 7) + blockIdx.x] = row_part[r][0] + row_part[r][1];
    quantize_tile_cols(tdg, dg_qt, dg_sct, 0, r0, c0, rows_cap);
    quantize_tile_cols(tdu, du_qt, du_sct, 0, r0, c0, rows_cap);
}

// row_grad[row] = sum over the column blocks of partials[row, :], in block order (fixed, reproducible)
__global__ void row_sum_kernel(const float* __restrict__ partials, int nblk, RowWindow win, float* __restrict__ out) {
    const int rows = win.num_rows ? min(max(*win.num_rows, 0), win.end) : win.end;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x + win.begin; row < rows;
         row += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float s = 0.0f;
        for (int b = 0; b < nblk; ++b) s += partials[row * nblk + b];
        out[row] = s;
    }
}

}  // namespace

namespace {
bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }
int check_window(const char* who, int row_begin, int* row_end, int64_t rows) {
    if (*row_end <= 0) *row_end = static_cast<int>(rows);
    MOKB_REQUIRE(row_begin >= 0 && row_begin % 128 == 0 && *row_end % 128 == 0 && row_begin <= *row_end && *row_end - row_begin <= rows,
                 "%s: bad row window [%d, %d) for %lld rows", who, row_begin, *row_end, static_cast<long long>(rows));
    return MOKB_OK;
}
}  // namespace

int quantize_impl(const void* x_bf16, int64_t E, int64_t M, int64_t N, const int32_t* num_rows, int row_begin, int row_end,
                  void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, cudaStream_t stream, int blocks, int32_t* done_counter) {
    TraceScope trace(stream, "quantize", row_begin);
    MOKB_REQUIRE(x_bf16 != nullptr, "mxfp8_quantize: null input");
    MOKB_REQUIRE(E > 0 && M > 0 && N > 0 && M % 128 == 0 && N % 128 == 0, "mxfp8_quantize: M and N must be positive multiples of 128");
    MOKB_REQUIRE((x_fp8 == nullptr) == (x_sc == nullptr) && (x_fp8_t == nullptr) == (x_sc_t == nullptr),
                 "mxfp8_quantize: data and scale outputs go together");
    MOKB_REQUIRE(x_fp8 || x_fp8_t, "mxfp8_quantize: at least one quantised layout must be requested");
    MOKB_REQUIRE(aligned32(x_bf16) && aligned32(x_fp8) && aligned32(x_fp8_t), "mxfp8_quantize: tensors must be 32-byte aligned");
    MOKB_TRY(check_window("mxfp8_quantize", row_begin, &row_end, M));
    if (row_begin == row_end) return MOKB_OK;
    if (x_fp8 == nullptr && E == 1 && done_counter == nullptr) {
        const int64_t ct = ((row_end - row_begin) / 128) * (N / CTILE_COLS);
        if (blocks <= 0) blocks = static_cast<int>(ct < 8ll * sm_count() ? ct : 8ll * sm_count());
        share_sms_with_gemm(quantize_cols_kernel);
        quantize_cols_kernel<<<static_cast<unsigned>(blocks), 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x_bf16), M, N,
                                                                                RowWindow{num_rows, row_begin, row_end},
                                                                                static_cast<uint8_t*>(x_fp8_t), static_cast<uint8_t*>(x_sc_t));
        MOKB_CUDA(cudaGetLastError());
        note_launch();
        return MOKB_OK;
    }
    const int64_t tiles = E * ((row_end - row_begin) / 128) * (N / 128);
    if (blocks <= 0) blocks = static_cast<int>(tiles < 16ll * sm_count() ? tiles : 16ll * sm_count());
    share_sms_with_gemm(quantize_kernel);
    quantize_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x_bf16), E, M, N,
                                                                       RowWindow{num_rows, row_begin, row_end},
                                                                       static_cast<uint8_t*>(x_fp8), static_cast<uint8_t*>(x_sc),
                                                                       static_cast<uint8_t*>(x_fp8_t), static_cast<uint8_t*>(x_sc_t), done_counter);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

int swiglu_bwd_quant_impl(const void* gate_q, const void* gate_sc, const void* up_q, const void* up_sc, const void* d_hidden,
                          int64_t rows_cap, int64_t I, const int32_t* num_rows, int row_begin, int row_end, int has_limit, float limit,
                          const float* row_scale, void* dg_q, void* dg_sc, void* dg_qt, void* dg_sct,
                          void* du_q, void* du_sc, void* du_qt, void* du_sct, float* partials, float* row_grad,
                          cudaStream_t stream) {
    TraceScope trace(stream, "swiglu_bwd_quant", row_begin);
    MOKB_REQUIRE(gate_q && gate_sc && up_q && up_sc && d_hidden && dg_q && dg_sc && dg_qt && dg_sct && du_q && du_sc && du_qt && du_sct,
                 "swiglu_bwd_quant: null pointer");
    MOKB_REQUIRE((partials == nullptr) == (row_grad == nullptr), "swiglu_bwd_quant: partials and row_grad go together");
    MOKB_REQUIRE(rows_cap > 0 && rows_cap % 128 == 0 && I > 0 && I % 128 == 0 && rows_cap / 128 <= 65535, "swiglu_bwd_quant: bad sizes");
    MOKB_REQUIRE(aligned32(gate_q) && aligned32(up_q) && aligned32(d_hidden) && aligned32(dg_q) && aligned32(dg_qt) && aligned32(du_q) &&
                 aligned32(du_qt), "swiglu_bwd_quant: tensors must be 32-byte aligned");
    MOKB_TRY(check_window("swiglu_bwd_quant", row_begin, &row_end, rows_cap));
    if (row_begin == row_end) return MOKB_OK;
    const size_t smem = 2 * TILE_WORDS * sizeof(uint32_t);
    MOKB_CUDA(cudaFuncSetAttribute(swiglu_bwd_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const RowWindow win{num_rows, row_begin, row_end};
    const dim3 grid(static_cast<unsigned>(I / 128), static_cast<unsigned>((row_end - row_begin) / 128));
    share_sms_with_gemm(swiglu_bwd_quant_kernel);
    swiglu_bwd_quant_kernel<<<grid, 256, smem, stream>>>(
        static_cast<const uint8_t*>(gate_q), static_cast<const uint8_t*>(gate_sc), static_cast<const uint8_t*>(up_q),
        static_cast<const uint8_t*>(up_sc), static_cast<const __nv_bfloat16*>(d_hidden), rows_cap, I, win, Clamp{has_limit, limit},
        row_scale, static_cast<uint8_t*>(dg_q), static_cast<uint8_t*>(dg_sc), static_cast<uint8_t*>(dg_qt), static_cast<uint8_t*>(dg_sct),
        static_cast<uint8_t*>(du_q), static_cast<uint8_t*>(du_sc), static_cast<uint8_t*>(du_qt), static_cast<uint8_t*>(du_sct), partials);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    if (row_grad) {
        const int blocks = min(sm_count() * 4, (row_end - row_begin + 255) / 256);
        row_sum_kernel<<<blocks, 256, 0, stream>>>(partials, static_cast<int>(I / 128), win, row_grad);
        MOKB_CUDA(cudaGetLastError());
        note_launch();
    }
    return MOKB_OK;
}

}  // namespace mokb

using namespace mokb;

extern "C" int mokb_mxfp8_quantize(const void* x_bf16, int64_t E, int64_t M, int64_t N,
                                   void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, void* stream) {
    return quantize_impl(x_bf16, E, M, N, nullptr, 0, 0, x_fp8, x_sc, x_fp8_t, x_sc_t, static_cast<cudaStream_t>(stream));
}
