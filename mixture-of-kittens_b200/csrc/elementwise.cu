// HBM-bound element-wise kernels of the layer: SwiGLU forward/backward and the
// two epilogues that add the shared expert to the (weighted) routed rows.
// All of them move 16-byte vectors, one per thread per access, coalesced.
#include "common.cuh"

namespace mokb {
namespace {

struct Clamp {
    int on;
    float limit;
};

__device__ __forceinline__ float silu_mul(float g, float u, const Clamp& c) {
    if (c.on) {
        g = fminf(g, c.limit);
        u = fminf(fmaxf(u, -c.limit), c.limit);
    }
    return g / (1.0f + __expf(-g)) * u;
}

// hidden = bf16(silu(gate) * up)      (reference: csrc/megakernel/swiglu.cuh:135-168)
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ hidden,
                                  const int32_t* __restrict__ num_rows, int64_t max_rows, int vec_per_row, Clamp c) {
    int64_t rows = num_rows ? *num_rows : max_rows;
    if (rows > max_rows || rows < 0) rows = 0;
    const int64_t n = rows * vec_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint4 g = gate[i], u = up[i];
        const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
        const uint32_t* upp = reinterpret_cast<const uint32_t*>(&u);
        uint4 h;
        uint32_t* hp = reinterpret_cast<uint32_t*>(&h);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 gf = unpack_bf16(gp[k]), uf = unpack_bf16(upp[k]);
            hp[k] = pack_bf16(silu_mul(gf.x, uf.x, c), silu_mul(gf.y, uf.y, c));
        }
        hidden[i] = h;
    }
}

// d_gate, d_up and the un-rounded hidden of one element (reference: swiglu.cuh:1-36).
__device__ __forceinline__ float swiglu_bwd_one(float g, float u, float dh, const Clamp& c, float* d_gate, float* d_up) {
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
    *d_gate = g_ok ? dsilu * u * dh : 0.0f;
    *d_up = u_ok ? silu * dh : 0.0f;
    return silu * u;
}

// One warp per row; the per-row sum of d_hidden * hidden / w is reduced in a
// fixed order (lane-strided partials, then an xor tree), so it is bit-reproducible.
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                  const uint4* __restrict__ d_hidden, uint4* __restrict__ d_gate, uint4* __restrict__ d_up,
                                  const float* __restrict__ row_scale, float* __restrict__ row_grad_out,
                                  const int32_t* __restrict__ num_rows, int64_t max_rows, int vec_per_row, Clamp c) {
    int64_t rows = num_rows ? *num_rows : max_rows;
    if (rows > max_rows || rows < 0) rows = 0;
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const int64_t nwarps = static_cast<int64_t>(gridDim.x) * wpb;
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * wpb + (threadIdx.x >> 5); row < rows; row += nwarps) {
        float inv_w = 1.0f;
        if (row_grad_out) {
            const float w = row_scale ? row_scale[row] : 1.0f;
            inv_w = w > 0.0f ? 1.0f / w : 0.0f;
        }
        float partial = 0.0f;
        const int64_t base = row * vec_per_row;
        for (int v = lane; v < vec_per_row; v += 32) {
            const uint4 g = gate[base + v], u = up[base + v], dh = d_hidden[base + v];
            const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
            const uint32_t* upp = reinterpret_cast<const uint32_t*>(&u);
            const uint32_t* dp = reinterpret_cast<const uint32_t*>(&dh);
            uint4 og, ou;
            uint32_t* ogp = reinterpret_cast<uint32_t*>(&og);
            uint32_t* oup = reinterpret_cast<uint32_t*>(&ou);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 gf = unpack_bf16(gp[k]), uf = unpack_bf16(upp[k]), df = unpack_bf16(dp[k]);
                float dg0, du0, dg1, du1;
                const float h0 = swiglu_bwd_one(gf.x, uf.x, df.x, c, &dg0, &du0);
                const float h1 = swiglu_bwd_one(gf.y, uf.y, df.y, c, &dg1, &du1);
                partial += df.x * inv_w * h0 + df.y * inv_w * h1;
                ogp[k] = pack_bf16(dg0, dg1);
                oup[k] = pack_bf16(du0, du1);
            }
            d_gate[base + v] = og;
            d_up[base + v] = ou;
        }
        if (row_grad_out) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, o);
            if (lane == 0) row_grad_out[row] = partial;
        }
    }
}

template <int W>
__device__ __forceinline__ void ld_words(const uint32_t* p, uint32_t (&v)[W]) {
    if (W == 8) {
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]),
                     "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p));
    } else {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
}
template <int W>
__device__ __forceinline__ void st_words(uint32_t* p, const uint32_t (&v)[W]) {
    if (W == 8) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                     "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
    } else {
        *reinterpret_cast<uint4*>(p) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// out[t] = bf16(shared[t] + sum_k w[t,k] * routed[t*K+k]), fp32, k ascending
// (reference: csrc/utils.cuh:43-95 and 140-176; WEIGHTED=false is the backward epilogue).
// One thread per W packed bf16 pairs of a token (W = 8: 32-byte accesses); the routed rows of up to eight
// routes are requested before the first one is used, so a thread keeps up to 256 bytes in flight.
template <bool WEIGHTED, int W>
__global__ void __launch_bounds__(256, 2) epilogue_kernel(const uint32_t* __restrict__ shared, const uint32_t* __restrict__ routed,
                                const float* __restrict__ weights, uint32_t* __restrict__ out,
                                int64_t tokens, int items_per_row, int topk) {
    const int64_t n = tokens * items_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t row_words = static_cast<int64_t>(items_per_row) * W;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t t = i / items_per_row;
        const int v = static_cast<int>(i - t * items_per_row);
        uint32_t s[W];
        ld_words<W>(shared + i * W, s);
        float acc[2 * W];
#pragma unroll
        for (int k = 0; k < W; ++k) {
            const float2 f = unpack_bf16(s[k]);
            acc[2 * k] = f.x;
            acc[2 * k + 1] = f.y;
        }
        const uint32_t* rrow = routed + (t * topk) * row_words + static_cast<int64_t>(v) * W;
        for (int k0 = 0; k0 < topk; k0 += 8) {
            uint32_t r[8][W];
            float w[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (k0 + u < topk) {
                    ld_words<W>(rrow + static_cast<int64_t>(k0 + u) * row_words, r[u]);
                    w[u] = WEIGHTED ? __ldg(weights + t * topk + k0 + u) : 1.0f;
                }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (k0 + u >= topk) continue;
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    const float2 f = unpack_bf16(r[u][k]);
                    if (WEIGHTED) {
                        acc[2 * k] = acc[2 * k] + f.x * w[u];      // k ascending, as the reference does
                        acc[2 * k + 1] = acc[2 * k + 1] + f.y * w[u];
                    } else {
                        acc[2 * k] += f.x;
                        acc[2 * k + 1] += f.y;
                    }
                }
            }
        }
        uint32_t o[W];
#pragma unroll
        for (int k = 0; k < W; ++k) o[k] = pack_bf16(acc[2 * k], acc[2 * k + 1]);
        st_words<W>(out + i * W, o);
    }
}

template <bool WEIGHTED>
int launch_epilogue(const void* shared, const void* routed, const float* weights, void* out, int64_t tokens, int64_t hidden, int topk,
                    cudaStream_t stream) {
    const bool wide = hidden % 16 == 0 && ((reinterpret_cast<uintptr_t>(shared) | reinterpret_cast<uintptr_t>(routed) |
                                            reinterpret_cast<uintptr_t>(out)) & 31) == 0;
    const int items = static_cast<int>(hidden / (wide ? 16 : 8));
    const int64_t work = tokens * items;
    int64_t blocks = (work + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const uint32_t* sp = static_cast<const uint32_t*>(shared);
    const uint32_t* rp = static_cast<const uint32_t*>(routed);
    uint32_t* op = static_cast<uint32_t*>(out);
    if (wide) epilogue_kernel<WEIGHTED, 8><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(sp, rp, weights, op, tokens, items, topk);
    else epilogue_kernel<WEIGHTED, 4><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(sp, rp, weights, op, tokens, items, topk);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

int grid_for(int64_t work_items, int threads) {
    int64_t blocks = (work_items + threads - 1) / threads;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" int mokb_swiglu_fwd(const void* gate, const void* up, void* hidden, const int32_t* num_rows, int64_t max_rows,
                               int64_t cols, int has_limit, float limit, void* stream) {
    MOKB_REQUIRE(gate && up && hidden, "swiglu_fwd: null pointer");
    MOKB_REQUIRE(max_rows >= 0 && cols > 0 && cols % 8 == 0, "swiglu_fwd: bad sizes");
    if (max_rows == 0) return MOKB_OK;
    Clamp c{has_limit, limit};
    const int vec = static_cast<int>(cols / 8);
    swiglu_fwd_kernel<<<grid_for(max_rows * vec, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<uint4*>(hidden), num_rows, max_rows, vec, c);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

extern "C" int mokb_swiglu_bwd(const void* gate, const void* up, const void* d_hidden, void* d_gate, void* d_up,
                               const float* row_scale, float* row_grad_out, const int32_t* num_rows,
                               int64_t max_rows, int64_t cols, int has_limit, float limit, void* stream) {
    TraceScope trace(static_cast<cudaStream_t>(stream), "swiglu_bwd");
    MOKB_REQUIRE(gate && up && d_hidden && d_gate && d_up, "swiglu_bwd: null pointer");
    MOKB_REQUIRE(max_rows >= 0 && cols > 0 && cols % 8 == 0, "swiglu_bwd: bad sizes");
    if (max_rows == 0) return MOKB_OK;
    Clamp c{has_limit, limit};
    const int vec = static_cast<int>(cols / 8);
    swiglu_bwd_kernel<<<grid_for(max_rows * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), static_cast<const uint4*>(d_hidden),
        static_cast<uint4*>(d_gate), static_cast<uint4*>(d_up), row_scale, row_grad_out, num_rows, max_rows, vec, c);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

extern "C" int mokb_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights,
                                 void* output, int64_t num_local_tokens, int64_t hidden, int topk, void* stream) {
    TraceScope trace(static_cast<cudaStream_t>(stream), "fwd_epilogue");
    MOKB_REQUIRE(y_shared && combine_buffer && topk_weights && output, "fwd_epilogue: null pointer");
    MOKB_REQUIRE(num_local_tokens > 0 && hidden > 0 && hidden % 8 == 0 && topk > 0 && topk <= 255, "fwd_epilogue: bad sizes");
    return launch_epilogue<true>(y_shared, combine_buffer, topk_weights, output, num_local_tokens, hidden, topk,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int mokb_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* d_x,
                                 int64_t num_local_tokens, int64_t hidden, int topk, void* stream) {
    TraceScope trace(static_cast<cudaStream_t>(stream), "bwd_epilogue");
    MOKB_REQUIRE(d_x_shared && d_x_routed_buffer && d_x, "bwd_epilogue: null pointer");
    MOKB_REQUIRE(num_local_tokens > 0 && hidden > 0 && hidden % 8 == 0 && topk > 0 && topk <= 255, "bwd_epilogue: bad sizes");
    return launch_epilogue<false>(d_x_shared, d_x_routed_buffer, nullptr, d_x, num_local_tokens, hidden, topk,
                                  static_cast<cudaStream_t>(stream));
}
