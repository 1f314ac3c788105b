// MXFP8 quantiser: bf16 -> E4M3 with one E8M0 scale per 32 elements, in the
// row direction ("normal") and/or the column direction ("transposed": the
// quantisation of x^T), scales laid out in the 32x16-byte tiles that
// tcgen05 block-scaled MMA consumes.
// Reference: csrc/mxfp8.cuh:45-72 (one block), :92-186 (tile), :188-278 (kernel, host).
#include "common.cuh"

namespace mokb {
namespace {

constexpr int TILE = 128;
constexpr int PITCH = TILE + 2;   // bf16 elements per smem row: odd word pitch, conflict-free column reads

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

// grid (N/128, M/128, E), 256 threads: one 128x128 tile per CTA.
__global__ void __launch_bounds__(256) quantize_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t N,
                                                       uint8_t* __restrict__ q, uint8_t* __restrict__ sc,
                                                       uint8_t* __restrict__ qt, uint8_t* __restrict__ sct) {
    __shared__ __nv_bfloat16 tile[TILE * PITCH];
    const int64_t e = blockIdx.z;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * TILE, c0 = static_cast<int64_t>(blockIdx.x) * TILE;
    const __nv_bfloat16* src = x + (e * M + r0) * N + c0;
    const int t = threadIdx.x;

    // load the tile: 16 threads x 16 B per row
    for (int i = t; i < TILE * 16; i += 256) {
        const int r = i >> 4, v = i & 15;
        const uint4 val = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * N + v * 8);
        uint32_t* d = reinterpret_cast<uint32_t*>(&tile[r * PITCH + v * 8]);
        d[0] = val.x; d[1] = val.y; d[2] = val.z; d[3] = val.w;
    }
    __syncthreads();

    if (q) {   // rows of x: item = (row, block of 32 columns)
        for (int item = t; item < TILE * 4; item += 256) {
            const int r = item >> 2, kb = item & 3;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[r * PITCH + kb * 32 + i]);
            uint32_t out[8];
            const uint32_t byte = quantize_block(v, out);
            uint4* dst = reinterpret_cast<uint4*>(q + (e * M + r0 + r) * N + c0 + kb * 32);
            dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
            dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
            sc[scale_offset(e * M + r0 + r, (c0 >> 5) + kb, N >> 7)] = static_cast<uint8_t>(byte);
        }
    }
    if (qt) {  // rows of x^T: item = (column c, block of 32 rows)
        for (int item = t; item < TILE * 4; item += 256) {
            const int c = item & 127, kb = item >> 7;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __bfloat162float(tile[(kb * 32 + i) * PITCH + c]);
            uint32_t out[8];
            const uint32_t byte = quantize_block(v, out);
            uint4* dst = reinterpret_cast<uint4*>(qt + (e * N + c0 + c) * M + r0 + kb * 32);
            dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
            dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
            sct[scale_offset(e * N + c0 + c, (r0 >> 5) + kb, M >> 7)] = static_cast<uint8_t>(byte);
        }
    }
}

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" int mokb_mxfp8_quantize(const void* x_bf16, int64_t E, int64_t M, int64_t N,
                                   void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, void* stream) {
    MOKB_REQUIRE(x_bf16 != nullptr, "mxfp8_quantize: null input");
    MOKB_REQUIRE(E > 0 && M > 0 && N > 0 && M % 128 == 0 && N % 128 == 0, "mxfp8_quantize: M and N must be positive multiples of 128");
    MOKB_REQUIRE((x_fp8 == nullptr) == (x_sc == nullptr) && (x_fp8_t == nullptr) == (x_sc_t == nullptr),
                 "mxfp8_quantize: data and scale outputs go together");
    MOKB_REQUIRE(x_fp8 || x_fp8_t, "mxfp8_quantize: at least one quantised layout must be requested");
    MOKB_REQUIRE(E <= 65535 && M / 128 <= 65535, "mxfp8_quantize: tensor too large for one launch");
    const dim3 grid(static_cast<unsigned>(N / 128), static_cast<unsigned>(M / 128), static_cast<unsigned>(E));
    quantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x_bf16), M, N, static_cast<uint8_t*>(x_fp8), static_cast<uint8_t*>(x_sc),
        static_cast<uint8_t*>(x_fp8_t), static_cast<uint8_t*>(x_sc_t));
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}
