// Device helpers of the MXFP8 codec shared by the quantising kernels and the MXFP8 GEMM epilogue:
// E4M3 data with one E8M0 scale per 32 elements (reference: csrc/mxfp8.cuh:45-90, 184).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace mokb {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// running per-half maximum of |x| over packed bf16 pairs
__device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t w) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&m),
                                     __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w)));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// block maximum -> E8M0 scale byte and the exact reciprocal of the scale (csrc/mxfp8.cuh:45-60):
// scale = max(amax / 448, 1e-12) rounded up to a power of two
__device__ __forceinline__ uint32_t scale_byte(float amax, float* inv) {
    const float scale = fmaxf(amax * 0.002232142857f, 0.000000000001f);
    uint16_t sc2;
    asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(sc2) : "f"(scale), "f"(scale));
    const uint32_t byte = sc2 & 0xFFu;
    *inv = __uint_as_float((254u - byte) << 23);
    return byte;
}

// four floats -> four E4M3 bytes (a in the lowest byte), round to nearest even, saturating (csrc/mxfp8.cuh:62-72)
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
    asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ void st_global_32B(void* p, const uint32_t (&v)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void ld_global_32B(const void* p, uint32_t (&v)[8]) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]),
                 "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p));
}

// byte offset of the scale of (row r, 32-element block kb) of a [rows, cols] matrix in the packed
// [rows/128, cols/128, 32, 16] layout (csrc/mxfp8.cuh:184)
__device__ __forceinline__ size_t scale_offset(int64_t r, int64_t kb, int64_t col_tiles) {
    const int64_t rt = r >> 7, ri = r & 127, ct = kb >> 2, ki = kb & 3;
    return static_cast<size_t>((rt * col_tiles + ct) * 512 + (ri & 31) * 16 + (ri >> 5) * 4 + ki);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

}  // namespace mokb
