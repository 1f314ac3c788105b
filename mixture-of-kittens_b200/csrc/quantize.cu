// MXFP8 codec kernels: bf16 -> E4M3 with one E8M0 scale per 32 elements, along rows
// ("normal") and/or along columns ("transposed": the quantisation of x^T), scales laid out
// in the 32 x 16-byte tiles that tcgen05 block-scaled MMA consumes.
//   quantize_kernel         plain quantiser            (reference: csrc/mxfp8.cuh:188-278)
//   swiglu_fwd_quant_kernel SwiGLU forward + quantise  (reference: csrc/megakernel/swiglu.cuh:38-207)
//   swiglu_bwd_quant_kernel de-quantise saved gate/up, SwiGLU backward, router-gradient partials,
//                           quantise d_gate / d_up      (reference: swiglu.cuh:209-566)
// One 128 x 128 tile per CTA, staged in shared memory with an odd word pitch so that both the
// row-wise and the column-wise passes read it without bank conflicts.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mokb {
namespace {

constexpr int TILE = 128;
constexpr int PITCH = TILE + 2;   // bf16 elements per smem row
constexpr int TILE_ELEMS = TILE * PITCH;

// 32 values -> 32 E4M3 bytes + scale byte (csrc/mxfp8.cuh:45-72)
__device__ __forceinline__ uint32_t quantize_block(const float (&v)[32], uint32_t (&out)[8]) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const float scale = fmaxf(amax * 0.002232142857f, 0.000000000001f);
    uint16_t sc2;
    asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(sc2) : "f"(scale), "f"(scale));
    const uint32_t byte = sc2 & 0xFFu;
    const float inv = __uint_as_float((254u - byte) << 23);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint16_t lo, hi;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(v[4 * i] * inv), "f"(v[4 * i + 1] * inv));
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(v[4 * i + 2] * inv), "f"(v[4 * i + 3] * inv));
        out[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    return byte;
}

// byte offset of the scale of (row r, 32-element block kb) of a [rows, cols] matrix in the packed
// [rows/128, cols/128, 32, 16] layout (csrc/mxfp8.cuh:184)
__device__ __forceinline__ size_t scale_offset(int64_t r, int64_t kb, int64_t col_tiles) {
    const int64_t rt = r >> 7, ri = r & 127, ct = kb >> 2, ki = kb & 3;
    return static_cast<size_t>((rt * col_tiles + ct) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + ki);
}

// Row-wise quantisation of a staged tile into q [rows, cols] (+ scales): item = (row, block of 32 columns).
__device__ __forceinline__ void quantize_tile_rows(const __nv_bfloat16* tile, uint8_t* q, uint8_t* sc, int64_t row_base,
                                                   int64_t r0, int64_t c0, int64_t cols) {
    for (int item = threadIdx.x; item < TILE * 4; item += blockDim.x) {
        const int r = item >> 2, kb = item & 3;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[r * PITCH + kb * 32 + i]);
        uint32_t out[8];
        const uint32_t byte = quantize_block(v, out);
        uint4* dst = reinterpret_cast<uint4*>(q + (row_base + r0 + r) * cols + c0 + kb * 32);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
        sc[scale_offset(row_base + r0 + r, (c0 >> 5) + kb, cols >> 7)] = static_cast<uint8_t>(byte);
    }
}

// Column-wise quantisation into qt [cols, rows] (+ scales): item = (column, block of 32 rows).
__device__ __forceinline__ void quantize_tile_cols(const __nv_bfloat16* tile, uint8_t* qt, uint8_t* sct, int64_t col_base,
                                                   int64_t r0, int64_t c0, int64_t rows) {
    for (int item = threadIdx.x; item < TILE * 4; item += blockDim.x) {
        const int c = item & 127, kb = item >> 7;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[(kb * 32 + i) * PITCH + c]);
        uint32_t out[8];
        const uint32_t byte = quantize_block(v, out);
        uint4* dst = reinterpret_cast<uint4*>(qt + (col_base + c0 + c) * rows + r0 + kb * 32);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
        sct[scale_offset(col_base + c0 + c, (r0 >> 5) + kb, rows >> 7)] = static_cast<uint8_t>(byte);
    }
}

__device__ __forceinline__ void load_tile_bf16(__nv_bfloat16* tile, const __nv_bfloat16* src, int64_t ld) {
    for (int i = threadIdx.x; i < TILE * 16; i += blockDim.x) {
        const int r = i >> 4, v = i & 15;
        const uint4 val = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * ld + v * 8);
        uint32_t* d = reinterpret_cast<uint32_t*>(&tile[r * PITCH + v * 8]);
        d[0] = val.x; d[1] = val.y; d[2] = val.z; d[3] = val.w;
    }
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ int live_rows(const int32_t* num_rows, int64_t cap) {
    if (!num_rows) return static_cast<int>(cap);
    const int n = *num_rows;
    return (n < 0 || n > cap) ? 0 : n;
}

// rows [begin, min(end, *num_rows)) of a tensor with `cap` rows; the grid's y index counts 128-row tiles from `begin`
struct RowWindow {
    const int32_t* num_rows;
    int begin, end;
};
__device__ __forceinline__ bool tile_in_window(const RowWindow& w, int64_t cap, int64_t* r0) {
    *r0 = static_cast<int64_t>(blockIdx.y) * TILE + w.begin;
    const int live = min(live_rows(w.num_rows, cap), w.end);
    return *r0 < live;
}

// grid (N/128, M/128, E), 256 threads.
__global__ void __launch_bounds__(256) quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t N,
                                                       RowWindow win,
                                                       uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                                       uint8_t* __restrict__ qt, uint8_t* __restrict__ sct) {
    __shared__ __nv_bfloat16 tile[TILE_ELEMS];
    const int64_t e = blockIdx.z;
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * TILE;
    int64_t r0;
    if (!tile_in_window(win, M, &r0)) return;
    load_tile_bf16(tile, x + (e * M + r0) * N + c0, N);
    __syncthreads();
    if (q) quantize_tile_rows(tile, q, sc, e * M, r0, c0, N);
    if (qt) quantize_tile_cols(tile, qt, sct, e * N, r0, c0, M);
}

struct Clamp {
    int on;
    float limit;
};

// gate, up [rows, I] bf16 -> gate_q, up_q, hidden_q (row-wise) and hidden_qt (column-wise).
// grid (I/128, rows_cap/128), 256 threads, 3 staged tiles.
__global__ void __launch_bounds__(256) swiglu_fwd_quant_kernel(
    const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, int64_t rows_cap, int64_t I,
    RowWindow win, Clamp c,
    uint8_t* gate_q, uint8_t* gate_sc, uint8_t* up_q, uint8_t* up_sc,
    uint8_t* hid_q, uint8_t* hid_sc, uint8_t* hid_qt, uint8_t* hid_sct) {
    extern __shared__ __nv_bfloat16 sm[];
    __nv_bfloat16 *tg = sm, *tu = sm + TILE_ELEMS, *th = sm + 2 * TILE_ELEMS;
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * TILE;
    int64_t r0;
    if (!tile_in_window(win, rows_cap, &r0)) return;
    load_tile_bf16(tg, gate + r0 * I + c0, I);
    load_tile_bf16(tu, up + r0 * I + c0, I);
    __syncthreads();
    for (int i = threadIdx.x; i < TILE * TILE; i += blockDim.x) {
        const int r = i >> 7, col = i & 127;
        float g = __bfloat162float(tg[r * PITCH + col]), u = __bfloat162float(tu[r * PITCH + col]);
        if (c.on) {
            g = fminf(g, c.limit);
            u = fminf(fmaxf(u, -c.limit), c.limit);
        }
        th[r * PITCH + col] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
    }
    __syncthreads();
    quantize_tile_rows(tg, gate_q, gate_sc, 0, r0, c0, I);
    quantize_tile_rows(tu, up_q, up_sc, 0, r0, c0, I);
    quantize_tile_rows(th, hid_q, hid_sc, 0, r0, c0, I);
    quantize_tile_cols(th, hid_qt, hid_sct, 0, r0, c0, rows_cap);
}

// Saved gate/up (E4M3 + scales), d_hidden bf16 -> d_gate, d_up (bf16 staged), their row-wise and
// column-wise quantisations, and the per-(row, 128-column block) router-gradient partial
// sum(d_hidden * silu(g) * u) / w.  grid (I/128, rows_cap/128), 256 threads.
__global__ void __launch_bounds__(256) swiglu_bwd_quant_kernel(
    const uint8_t* __restrict__ gate_q, const uint8_t* __restrict__ gate_sc, const uint8_t* __restrict__ up_q,
    const uint8_t* __restrict__ up_sc, const __nv_bfloat16* __restrict__ d_hidden, int64_t rows_cap, int64_t I,
    RowWindow win, Clamp c, const float* __restrict__ row_scale,
    uint8_t* dg_q, uint8_t* dg_sc, uint8_t* dg_qt, uint8_t* dg_sct,
    uint8_t* du_q, uint8_t* du_sc, uint8_t* du_qt, uint8_t* du_sct, float* __restrict__ partials) {
    extern __shared__ __nv_bfloat16 sm[];
    __nv_bfloat16 *tdh = sm, *tdg = sm + TILE_ELEMS, *tdu = sm + 2 * TILE_ELEMS;
    __shared__ float row_part[TILE][2];
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * TILE;
    int64_t r0;
    if (!tile_in_window(win, rows_cap, &r0)) return;
    load_tile_bf16(tdh, d_hidden + r0 * I + c0, I);
    __syncthreads();
    // two threads per row, 64 columns each (two scale blocks of 32)
    const int r = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int64_t row = r0 + r;
    const float w = row_scale ? row_scale[row] : 1.0f;
    const float inv_w = w > 0.0f ? 1.0f / w : 0.0f;
    float partial = 0.0f;
    for (int kb = half * 2; kb < half * 2 + 2; ++kb) {
        const float gs = __uint_as_float(static_cast<uint32_t>(gate_sc[scale_offset(row, (c0 >> 5) + kb, I >> 7)]) << 23);
        const float us = __uint_as_float(static_cast<uint32_t>(up_sc[scale_offset(row, (c0 >> 5) + kb, I >> 7)]) << 23);
        const uint4* gp = reinterpret_cast<const uint4*>(gate_q + row * I + c0 + kb * 32);
        const uint4* upp = reinterpret_cast<const uint4*>(up_q + row * I + c0 + kb * 32);
        uint4 gv[2] = {gp[0], gp[1]}, uv[2] = {upp[0], upp[1]};
        const uint8_t* gb = reinterpret_cast<const uint8_t*>(gv);
        const uint8_t* ub = reinterpret_cast<const uint8_t*>(uv);
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            float g = e4m3_to_float(gb[i]) * gs, u = e4m3_to_float(ub[i]) * us;
            const float dh = __bfloat162float(tdh[r * PITCH + kb * 32 + i]);
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
            tdg[r * PITCH + kb * 32 + i] = __float2bfloat16_rn(g_ok ? dsilu * u * dh : 0.0f);
            tdu[r * PITCH + kb * 32 + i] = __float2bfloat16_rn(u_ok ? silu * dh : 0.0f);
            partial += dh * inv_w * (silu * u);
        }
    }
    row_part[r][half] = partial;
    __syncthreads();
    if (partials && half == 0) partials[row * (I >> 7) + blockIdx.x] = row_part[r][0] + row_part[r][1];
    quantize_tile_rows(tdg, dg_q, dg_sc, 0, r0, c0, I);
    quantize_tile_rows(tdu, du_q, du_sc, 0, r0, c0, I);
    quantize_tile_cols(tdg, dg_qt, dg_sct, 0, r0, c0, rows_cap);
    quantize_tile_cols(tdu, du_qt, du_sct, 0, r0, c0, rows_cap);
}

// row_grad[row] = sum over the column blocks of partials[row, :], in block order (fixed, reproducible)
__global__ void row_sum_kernel(const float* __restrict__ partials, int nblk, RowWindow win, int64_t rows_cap,
                               float* __restrict__ out) {
    const int rows = min(live_rows(win.num_rows, rows_cap), win.end);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x + win.begin; row < rows;
         row += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        float s = 0.0f;
        for (int b = 0; b < nblk; ++b) s += partials[row * nblk + b];
        out[row] = s;
    }
}

}  // namespace

int quantize_impl(const void* x_bf16, int64_t E, int64_t M, int64_t N, const int32_t* num_rows, int row_begin, int row_end,
                  void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, cudaStream_t stream) {
    if (row_end <= 0) row_end = static_cast<int>(M);
    MOKB_REQUIRE(row_begin >= 0 && row_begin % 128 == 0 && row_end % 128 == 0 && row_begin <= row_end && row_end <= M,
                 "mxfp8_quantize: bad row window");
    if (row_begin == row_end) return MOKB_OK;
    MOKB_REQUIRE(x_bf16 != nullptr, "mxfp8_quantize: null input");
    MOKB_REQUIRE(E > 0 && M > 0 && N > 0 && M % 128 == 0 && N % 128 == 0, "mxfp8_quantize: M and N must be positive multiples of 128");
    MOKB_REQUIRE((x_fp8 == nullptr) == (x_sc == nullptr) && (x_fp8_t == nullptr) == (x_sc_t == nullptr),
                 "mxfp8_quantize: data and scale outputs go together");
    MOKB_REQUIRE(x_fp8 || x_fp8_t, "mxfp8_quantize: at least one quantised layout must be requested");
    MOKB_REQUIRE(E <= 65535 && M / 128 <= 65535, "mxfp8_quantize: tensor too large for one launch");
    const dim3 grid(static_cast<unsigned>(N / 128), static_cast<unsigned>((row_end - row_begin) / 128), static_cast<unsigned>(E));
    quantize_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x_bf16), M, N, RowWindow{num_rows, row_begin, row_end},
                                              static_cast<uint8_t*>(x_fp8), static_cast<uint8_t*>(x_sc),
                                              static_cast<uint8_t*>(x_fp8_t), static_cast<uint8_t*>(x_sc_t));
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

int swiglu_fwd_quant_impl(const void* gate, const void* up, int64_t rows_cap, int64_t I, const int32_t* num_rows,
                          int row_begin, int row_end, int has_limit, float limit, void* gate_q, void* gate_sc, void* up_q, void* up_sc,
                          void* hid_q, void* hid_sc, void* hid_qt, void* hid_sct, cudaStream_t stream) {
    MOKB_REQUIRE(gate && up && gate_q && gate_sc && up_q && up_sc && hid_q && hid_sc && hid_qt && hid_sct, "swiglu_fwd_quant: null pointer");
    MOKB_REQUIRE(rows_cap > 0 && rows_cap % 128 == 0 && I > 0 && I % 128 == 0 && rows_cap / 128 <= 65535, "swiglu_fwd_quant: bad sizes");
    const size_t smem = 3 * TILE_ELEMS * sizeof(__nv_bfloat16);
    MOKB_CUDA(cudaFuncSetAttribute(swiglu_fwd_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (row_end <= 0) row_end = static_cast<int>(rows_cap);
    MOKB_REQUIRE(row_begin >= 0 && row_begin % 128 == 0 && row_end % 128 == 0 && row_begin <= row_end && row_end <= rows_cap,
                 "swiglu_fwd_quant: bad row window");
    if (row_begin == row_end) return MOKB_OK;
    const dim3 grid(static_cast<unsigned>(I / 128), static_cast<unsigned>((row_end - row_begin) / 128));
    swiglu_fwd_quant_kernel<<<grid, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up), rows_cap, I, RowWindow{num_rows, row_begin, row_end},
        Clamp{has_limit, limit},
        static_cast<uint8_t*>(gate_q), static_cast<uint8_t*>(gate_sc), static_cast<uint8_t*>(up_q), static_cast<uint8_t*>(up_sc),
        static_cast<uint8_t*>(hid_q), static_cast<uint8_t*>(hid_sc), static_cast<uint8_t*>(hid_qt), static_cast<uint8_t*>(hid_sct));
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

int swiglu_bwd_quant_impl(const void* gate_q, const void* gate_sc, const void* up_q, const void* up_sc, const void* d_hidden,
                          int64_t rows_cap, int64_t I, const int32_t* num_rows, int row_begin, int row_end, int has_limit, float limit,
                          const float* row_scale, void* dg_q, void* dg_sc, void* dg_qt, void* dg_sct,
                          void* du_q, void* du_sc, void* du_qt, void* du_sct, float* partials, float* row_grad,
                          cudaStream_t stream) {
    MOKB_REQUIRE(gate_q && gate_sc && up_q && up_sc && d_hidden && dg_q && dg_sc && dg_qt && dg_sct && du_q && du_sc && du_qt && du_sct,
                 "swiglu_bwd_quant: null pointer");
    MOKB_REQUIRE((partials == nullptr) == (row_grad == nullptr), "swiglu_bwd_quant: partials and row_grad go together");
    MOKB_REQUIRE(rows_cap > 0 && rows_cap % 128 == 0 && I > 0 && I % 128 == 0 && rows_cap / 128 <= 65535, "swiglu_bwd_quant: bad sizes");
    const size_t smem = 3 * TILE_ELEMS * sizeof(__nv_bfloat16);
    MOKB_CUDA(cudaFuncSetAttribute(swiglu_bwd_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (row_end <= 0) row_end = static_cast<int>(rows_cap);
    MOKB_REQUIRE(row_begin >= 0 && row_begin % 128 == 0 && row_end % 128 == 0 && row_begin <= row_end && row_end <= rows_cap,
                 "swiglu_bwd_quant: bad row window");
    if (row_begin == row_end) return MOKB_OK;
    const RowWindow win{num_rows, row_begin, row_end};
    const dim3 grid(static_cast<unsigned>(I / 128), static_cast<unsigned>((row_end - row_begin) / 128));
    swiglu_bwd_quant_kernel<<<grid, 256, smem, stream>>>(
        static_cast<const uint8_t*>(gate_q), static_cast<const uint8_t*>(gate_sc), static_cast<const uint8_t*>(up_q),
        static_cast<const uint8_t*>(up_sc), static_cast<const __nv_bfloat16*>(d_hidden), rows_cap, I, win, Clamp{has_limit, limit},
        row_scale, static_cast<uint8_t*>(dg_q), static_cast<uint8_t*>(dg_sc), static_cast<uint8_t*>(dg_qt), static_cast<uint8_t*>(dg_sct),
        static_cast<uint8_t*>(du_q), static_cast<uint8_t*>(du_sc), static_cast<uint8_t*>(du_qt), static_cast<uint8_t*>(du_sct), partials);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    if (row_grad) {
        const int blocks = min(sm_count() * 4, (row_end - row_begin + 255) / 256);
        row_sum_kernel<<<blocks, 256, 0, stream>>>(partials, static_cast<int>(I / 128), win, rows_cap, row_grad);
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
