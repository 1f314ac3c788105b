// Cross-GPU pieces of the layer, all over plain peer-to-peer loads and stores
// through NVLink/NVSwitch unicast addresses (no NCCL, no multicast object):
//   * route all-gather   (reference: csrc/utils.cuh:191-249, NVLS multicast store)
//   * device barrier     (reference: csrc/utils.cuh:251-299, multimem.red)
//   * dispatch = row pull from the token's home rank
//                        (reference: csrc/megakernel/dispatch_combine.cuh:1-150)
//   * combine  = row push into the home rank's [T*K, H] buffer
//                        (reference: dispatch_combine.cuh:152-266)
// With ep_size == 1 the same kernels run against the local pointers.
#include "common.cuh"
#include "mxfp8_codec.cuh"

namespace mokb {
namespace {

__device__ __forceinline__ void st_v4(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// W 32-bit words per access: 4 (16 bytes) or 8 (32 bytes: one full sector, half the instructions)
template <int W>
struct Words {
    uint32_t w[W];
};
template <int W>
__device__ __forceinline__ Words<W> ld_words(const void* p) {
    Words<W> v;
    if (W == 8) {
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]),
                     "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    } else {
        asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(p));
    }
    return v;
}
template <int W>
__device__ __forceinline__ void st_words(void* p, const Words<W>& v) {
    if (W == 8) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]),
                     "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7]) : "memory");
    } else {
        asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
    }
}

__global__ void all_gather_kernel(const uint4* __restrict__ src, PeerPtrs peers, int R, int rank, int64_t nvec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = src[i];
        for (int r = 0; r < R; ++r) st_v4(static_cast<uint4*>(peers.p[r]) + rank * nvec + i, v);
    }
}

// One CTA.  Thread r adds 1 to rank r's barrier word (release, system scope);
// thread 0 then waits until the local word reaches the new target.
__global__ void barrier_kernel(PeerPtrs peers, int R, int rank, int32_t* target, int32_t* status,
                               unsigned long long timeout_ns) {
    __shared__ int new_target;
    if (threadIdx.x == 0) {
        new_target = *target + R;
        *target = new_target;
    }
    __syncthreads();
    if (threadIdx.x < R) {
        __threadfence_system();
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peers.p[threadIdx.x]) : "memory");
    }
    if (threadIdx.x == 0) {
        const int32_t* mine = static_cast<const int32_t*>(peers.p[rank]);
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (uint32_t i = 0;; ++i) {
            int32_t v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v - new_target >= 0) break;
            if ((i & 63) == 63) {
                unsigned long long t1;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > timeout_ns) {
                    atomicCAS(status, MOKB_ST_OK, MOKB_ST_BARRIER_TIMEOUT);
                    break;
                }
                __nanosleep(100);
            }
        }
        __threadfence_system();
    }
}

// Row-wise MXFP8 form of the rows a dispatch pulls (QUANT variants): E4M3 bytes [rows, H] and packed scales.
struct RowQuant {
    uint8_t* q;
    uint8_t* sc;
    int col_tiles;          // H / 128
};

// One warp per schedule row, 16- or 32-byte accesses, four loads in flight per lane.  QUANT (32-byte accesses only):
// the row is also quantised along its columns from the registers it passes through -- a lane holds 16 consecutive
// values, two neighbouring lanes one 32-value block (the reference quantises the tile it has just pulled,
// csrc/megakernel/dispatch_combine.cuh:88-114; the values are those of quantize_kernel, byte for byte).
template <bool SCALE, int W, bool QUANT>
__global__ void __maxnreg__(64) dispatch_kernel(PeerPtrs src, PeerPtrs scale_src, const int32_t* __restrict__ peer_rank,
                                const int32_t* __restrict__ peer_token_idx, const int32_t* __restrict__ num_rows,
                                int max_rows, int row_begin, int row_end, int R, int row_divisor, int vec_per_row,
                                Words<W>* __restrict__ dst, float* __restrict__ row_scale_out, int32_t* done_counter, RowQuant rq,
                                IndexGuard guard) {
    int rows = num_rows ? *num_rows : max_rows;
    rows = rows < 0 ? 0 : (rows > max_rows ? 0 : rows);
    rows = min(rows, row_end);
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * warps_per_block;
    // The indices (and the remote scale) of a warp's next row are fetched while it moves the current one: three
    // dependent round trips (indices, scale over NVLink, data over NVLink) would otherwise sit in front of every row.
    int row = row_begin + warp;
    int pr_next = -1, tok_next = 0;
    float w_next = 1.f;
    auto fetch_indices = [&](int r) {
        pr_next = -1;
        if (r < rows) {
            pr_next = peer_rank[r];
            tok_next = peer_token_idx[r];
            if (pr_next >= 0 && pr_next < R && !index_ok(guard, tok_next, kBadIndexPull, r)) pr_next = -1;
            if (SCALE && pr_next >= 0 && pr_next < R) w_next = static_cast<const float*>(scale_src.p[pr_next])[tok_next];
        }
    };
    fetch_indices(row);
    for (; row < rows; row += nwarps) {
        const int pr = pr_next;
        const int tok = tok_next;
        const float w = SCALE ? w_next : 1.f;
        fetch_indices(row + nwarps);
        Words<W>* out = dst + static_cast<size_t>(row) * vec_per_row;
        if (pr < 0 || pr >= R) {      // padding row (or a rank outside the pointer list: treated as padding, never dereferenced)
            Words<W> zero;
#pragma unroll
            for (int k = 0; k < W; ++k) zero.w[k] = 0u;
            for (int v = lane; v < vec_per_row; v += 32) st_words<W>(out + v, zero);
            if (SCALE && lane == 0 && row_scale_out) row_scale_out[row] = 0.f;
            if (QUANT) {          // a zero row: zero bytes and the scale of an all-zero block
                float inv;
                const uint8_t zb = static_cast<uint8_t>(scale_byte(0.f, &inv));
                for (int v = lane; v < vec_per_row; v += 32) {
                    asm volatile("st.global.v4.u32 [%0], {%1, %1, %1, %1};" ::"l"(rq.q + static_cast<size_t>(row) * vec_per_row * 16 + v * 16), "r"(0u) : "memory");
                    if ((v & 1) == 0) rq.sc[scale_offset(row, v >> 1, rq.col_tiles)] = zb;
                }
            }
            continue;
        }
        const Words<W>* in = static_cast<const Words<W>*>(src.p[pr]) + static_cast<size_t>(tok / row_divisor) * vec_per_row;
        if (SCALE && lane == 0 && row_scale_out) row_scale_out[row] = w;
        // (every lane makes the same number of trips: the quantising variant shuffles between lanes inside)
        for (int vb = 0; vb < vec_per_row; vb += 128) {
            const int v0 = vb + lane;
            Words<W> r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (v0 + 32 * u < vec_per_row) r[u] = ld_words<W>(in + v0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const bool live = v0 + 32 * u < vec_per_row;
                if (live) {
                    if (SCALE) {
#pragma unroll
                        for (int k = 0; k < W; ++k) {
                            const float2 f = unpack_bf16(r[u].w[k]);
                            r[u].w[k] = pack_bf16(f.x * w, f.y * w);
                        }
                    }
                    st_words<W>(out + v0 + 32 * u, r[u]);
                }
                if (QUANT) {      // lanes 2j and 2j+1 hold one 32-value block (W = 8: 16 values per lane); whole warp
                    uint32_t m = 0u;
                    if (live) {
#pragma unroll
                        for (int k = 0; k < W; ++k) m = absmax2(m, r[u].w[k]);
                    }
                    float amax = fmaxf(bf16_lo(m), bf16_hi(m));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    if (live) {
                        float inv;
                        const uint32_t byte = scale_byte(amax, &inv);
                        const int v = v0 + 32 * u;
                        uint32_t o[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            o[k] = e4m3x4(bf16_lo(r[u].w[2 * k]) * inv, bf16_hi(r[u].w[2 * k]) * inv,
                                          bf16_lo(r[u].w[2 * k + 1]) * inv, bf16_hi(r[u].w[2 * k + 1]) * inv);
                        asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(rq.q + static_cast<size_t>(row) * vec_per_row * 16 + v * 16),
                                     "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                        if ((lane & 1) == 0) rq.sc[scale_offset(row, v >> 1, rq.col_tiles)] = static_cast<uint8_t>(byte);
                    }
                }
            }
        }
    }
    if (done_counter) {      // this block's rows of the window have landed: one arrival for whoever consumes them
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            red_release_gpu_add(done_counter, 1);
        }
    }
}

template <int W>
__global__ void combine_kernel(const Words<W>* __restrict__ src, PeerPtrs dst, PeerPtrs val_dst,
                               const int32_t* __restrict__ peer_rank, const int32_t* __restrict__ peer_token_idx,
                               const int32_t* __restrict__ num_rows, int max_rows, int row_begin, int row_end, int R,
                               int vec_per_row, const float* __restrict__ row_values, const int32_t* wait_counter,
                               int arrivals_per_row_block, int32_t* status, int index_limit) {
    int rows = num_rows ? *num_rows : max_rows;
    rows = rows < 0 ? 0 : (rows > max_rows ? 0 : rows);
    rows = min(rows, row_end);
    if (wait_counter) {
        // the rows come from a GEMM that is still running: wait (bounded) until every tile of this window is stored
        __shared__ int go;
        if (threadIdx.x == 0) {
            const int expected = ((rows - row_begin) / 256) * arrivals_per_row_block;
            go = expected <= 0 || flag_wait(wait_counter, expected, nullptr, status, kWaitWindowDone, row_begin / 256);
        }
        __syncthreads();
        if (!go) return;
    }
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int warp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * warps_per_block;
    for (int row = row_begin + warp; row < rows; row += nwarps) {
        const int pr = peer_rank[row];
        if (pr < 0 || pr >= R) continue;
        const int tok = peer_token_idx[row];
        if (!index_ok(IndexGuard{index_limit, status}, tok, kBadIndexPush, row)) continue;
        const Words<W>* in = src + static_cast<size_t>(row) * vec_per_row;
        Words<W>* out = static_cast<Words<W>*>(dst.p[pr]) + static_cast<size_t>(tok) * vec_per_row;
        for (int v0 = lane; v0 < vec_per_row; v0 += 128) {
            Words<W> r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (v0 + 32 * u < vec_per_row) r[u] = ld_words<W>(in + v0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (v0 + 32 * u < vec_per_row) st_words<W>(out + v0 + 32 * u, r[u]);
        }
        if (row_values && lane == 0) static_cast<float*>(val_dst.p[pr])[tok] = row_values[row];
    }
}

// 32-byte accesses need 32-byte aligned rows everywhere: the local buffer and every peer's
bool rows_aligned32(const void* local, const PeerPtrs& peers, int R, int64_t hidden) {
    if (hidden % 16 != 0 || (reinterpret_cast<uintptr_t>(local) & 31) != 0) return false;
    for (int r = 0; r < R; ++r)
        if ((reinterpret_cast<uintptr_t>(peers.p[r]) & 31) != 0) return false;
    return true;
}

int fill_peers(PeerPtrs* out, const uint64_t* host, int R, const char* what) {
    MOKB_REQUIRE(host != nullptr, "%s: null pointer list", what);
    for (int r = 0; r < kPeerMax; ++r) out->p[r] = nullptr;
    for (int r = 0; r < R; ++r) {
        MOKB_REQUIRE(host[r] != 0 && (host[r] & 15) == 0, "%s[%d] = 0x%llx is null or not 16-byte aligned", what, r,
                     (unsigned long long)host[r]);
        out->p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(host[r]));
    }
    return MOKB_OK;
}

unsigned long long g_barrier_timeout_ns = 10ull * 1000 * 1000 * 1000;

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" int mokb_set_barrier_timeout_ms(int ms) {
    MOKB_REQUIRE(ms > 0, "barrier timeout must be positive");
    g_barrier_timeout_ns = static_cast<unsigned long long>(ms) * 1000ull * 1000ull;
    return MOKB_OK;
}

extern "C" int mokb_all_gather_top_experts(const int32_t* top_experts, const uint64_t* gather_buffer_ptrs_host,
                                           int ep_size, int rank, int64_t numel, void* stream) {
    TraceScope trace(static_cast<cudaStream_t>(stream), "all_gather_top_experts");
    MOKB_REQUIRE(top_experts != nullptr, "all_gather_top_experts: null input");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP && rank >= 0 && rank < ep_size, "all_gather_top_experts: bad ep_size/rank");
    MOKB_REQUIRE(numel > 0 && numel % 4 == 0, "all_gather_top_experts: numel must be a positive multiple of 4");
    MOKB_REQUIRE((reinterpret_cast<uintptr_t>(top_experts) & 15) == 0, "all_gather_top_experts: input not 16-byte aligned");
    PeerPtrs peers;
    MOKB_TRY(fill_peers(&peers, gather_buffer_ptrs_host, ep_size, "gather_buffer_ptrs"));
    const int64_t nvec = numel / 4;
    const int threads = 256;
    int64_t blocks = (nvec + threads - 1) / threads;
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    all_gather_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(top_experts), peers, ep_size, rank, nvec);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

extern "C" int mokb_barrier_all(const uint64_t* barrier_ptrs_host, int ep_size, int rank, int32_t* target,
                                int32_t* status, void* stream) {
    TraceScope trace(static_cast<cudaStream_t>(stream), "barrier_all");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP && rank >= 0 && rank < ep_size, "barrier_all: bad ep_size/rank");
    MOKB_REQUIRE(target && status, "barrier_all: null pointer");
    PeerPtrs peers;
    MOKB_REQUIRE(barrier_ptrs_host != nullptr, "barrier_all: null pointer list");
    for (int r = 0; r < kPeerMax; ++r) peers.p[r] = nullptr;
    for (int r = 0; r < ep_size; ++r) {
        MOKB_REQUIRE(barrier_ptrs_host[r] != 0 && (barrier_ptrs_host[r] & 3) == 0, "barrier_all: bad pointer for rank %d", r);
        peers.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(barrier_ptrs_host[r]));
    }
    barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(peers, ep_size, rank, target, status, g_barrier_timeout_ns);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

namespace mokb {

int comm_default_blocks() { return sm_count() * 16; }

int dispatch_rows_impl(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                       const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin, int row_end,
                       int row_divisor, int64_t hidden, void* dst, const uint64_t* row_scale_ptrs_host,
                       float* row_scale_out, int blocks, cudaStream_t s, int32_t* done_counter, void* q_out, void* q_sc_out,
                       int64_t index_limit, int32_t* status) {
    TraceScope trace(s, row_scale_ptrs_host ? "dispatch_scaled" : "dispatch", row_begin);
    MOKB_REQUIRE((q_out == nullptr) == (q_sc_out == nullptr), "dispatch_rows: the quantised rows and their scales go together");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP, "dispatch_rows: bad ep_size");
    MOKB_REQUIRE(peer_rank && peer_token_idx && dst, "dispatch_rows: null pointer");
    MOKB_REQUIRE(max_rows >= 0 && row_divisor >= 1 && hidden > 0 && hidden % 8 == 0, "dispatch_rows: bad sizes");
    MOKB_REQUIRE(row_begin >= 0 && row_begin <= row_end, "dispatch_rows: bad row window");
    MOKB_REQUIRE(index_limit >= 0 && index_limit <= INT32_MAX && (index_limit == 0 || status != nullptr),
                 "dispatch_rows: index_limit needs a status word and must fit 31 bits");
    const IndexGuard guard{static_cast<int>(index_limit), status};
    MOKB_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, "dispatch_rows: dst not 16-byte aligned");
    PeerPtrs src, scale;
    MOKB_TRY(fill_peers(&src, src_ptrs_host, ep_size, "src_ptrs"));
    for (int r = 0; r < kPeerMax; ++r) scale.p[r] = nullptr;
    if (max_rows == 0 || row_begin >= max_rows) return MOKB_OK;
    // 128 threads: one warp per SM quarter, so that a block finds room beside a GEMM CTA whatever that kernel's warp count
    const int threads = 128;
    if (blocks <= 0) blocks = comm_default_blocks();
    const bool wide = rows_aligned32(dst, src, ep_size, hidden);
    const int vec = static_cast<int>(hidden / (wide ? 16 : 8));
    for (int r = 0; r < ep_size && row_scale_ptrs_host; ++r) {
        MOKB_REQUIRE(row_scale_ptrs_host[r] != 0, "dispatch_rows: null scale pointer for rank %d", r);
        scale.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(row_scale_ptrs_host[r]));
    }
    const RowQuant rq{static_cast<uint8_t*>(q_out), static_cast<uint8_t*>(q_sc_out), static_cast<int>(hidden / 128)};
    if (q_out) {
        MOKB_REQUIRE(wide && hidden % 128 == 0 && (reinterpret_cast<uintptr_t>(q_out) & 15) == 0,
                     "dispatch_rows: quantised output needs 32-byte aligned rows, hidden %% 128 == 0 and a 16-byte aligned buffer");
    }
#define MOKB_DISPATCH(SC, WW, QQ)                                                                                              \
    do {                                                                                                                       \
        share_sms_with_gemm(dispatch_kernel<SC, WW, QQ>);                                                                      \
        dispatch_kernel<SC, WW, QQ><<<blocks, threads, 0, s>>>(src, scale, peer_rank, peer_token_idx, num_rows, max_rows,      \
            row_begin, row_end, ep_size, row_divisor, vec, static_cast<Words<WW>*>(dst), SC ? row_scale_out : nullptr,         \
            done_counter, rq, guard);                                                                                          \
    } while (0)
    if (row_scale_ptrs_host) {
        if (q_out) MOKB_DISPATCH(true, 8, true);
        else if (wide) MOKB_DISPATCH(true, 8, false);
        else MOKB_DISPATCH(true, 4, false);
    } else {
        if (q_out) MOKB_DISPATCH(false, 8, true);
        else if (wide) MOKB_DISPATCH(false, 8, false);
        else MOKB_DISPATCH(false, 4, false);
    }
#undef MOKB_DISPATCH
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

int combine_rows_impl(const void* src, const uint64_t* dst_ptrs_host, int ep_size, const int32_t* peer_rank,
                      const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin, int row_end,
                      int64_t hidden, const float* row_values, const uint64_t* value_ptrs_host, int blocks, cudaStream_t s,
                      const int32_t* wait_counter, int arrivals_per_row_block, int32_t* status, int64_t index_limit) {
    TraceScope trace(s, "combine", row_begin);
    MOKB_REQUIRE(index_limit >= 0 && index_limit <= INT32_MAX && (index_limit == 0 || status != nullptr),
                 "combine_rows: index_limit needs a status word and must fit 31 bits");
    MOKB_REQUIRE(wait_counter == nullptr || (arrivals_per_row_block > 0 && status != nullptr && row_begin % 256 == 0),
                 "combine_rows: a wait counter needs arrivals_per_row_block, a status word and a window that starts on a 256-row block");
    MOKB_REQUIRE(ep_size >= 1 && ep_size <= MOKB_MAX_EP, "combine_rows: bad ep_size");
    MOKB_REQUIRE(src && peer_rank && peer_token_idx, "combine_rows: null pointer");
    MOKB_REQUIRE(max_rows >= 0 && hidden > 0 && hidden % 8 == 0, "combine_rows: bad sizes");
    MOKB_REQUIRE(row_begin >= 0 && row_begin <= row_end, "combine_rows: bad row window");
    MOKB_REQUIRE((row_values == nullptr) == (value_ptrs_host == nullptr), "combine_rows: row_values and value_ptrs go together");
    PeerPtrs dst, val;
    MOKB_TRY(fill_peers(&dst, dst_ptrs_host, ep_size, "dst_ptrs"));
    for (int r = 0; r < kPeerMax; ++r) val.p[r] = nullptr;
    if (value_ptrs_host)
        for (int r = 0; r < ep_size; ++r) {
            MOKB_REQUIRE(value_ptrs_host[r] != 0, "combine_rows: null value pointer for rank %d", r);
            val.p[r] = reinterpret_cast<void*>(static_cast<uintptr_t>(value_ptrs_host[r]));
        }
    if (max_rows == 0 || row_begin >= max_rows) return MOKB_OK;
    if (blocks <= 0) blocks = comm_default_blocks();
    share_sms_with_gemm(combine_kernel<8>);
    share_sms_with_gemm(combine_kernel<4>);
    if (rows_aligned32(src, dst, ep_size, hidden))
        combine_kernel<8><<<blocks, 128, 0, s>>>(static_cast<const Words<8>*>(src), dst, val, peer_rank, peer_token_idx, num_rows, max_rows,
                                                 row_begin, row_end, ep_size, static_cast<int>(hidden / 16), row_values, wait_counter,
                                                 arrivals_per_row_block, status, static_cast<int>(index_limit));
    else
        combine_kernel<4><<<blocks, 128, 0, s>>>(static_cast<const Words<4>*>(src), dst, val, peer_rank, peer_token_idx, num_rows, max_rows,
                                                 row_begin, row_end, ep_size, static_cast<int>(hidden / 8), row_values, wait_counter,
                                                 arrivals_per_row_block, status, static_cast<int>(index_limit));
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

}  // namespace mokb

extern "C" int mokb_dispatch_rows(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                                  const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows,
                                  int row_divisor, int64_t hidden, void* dst,
                                  const uint64_t* row_scale_ptrs_host, float* row_scale_out, void* stream) {
    return dispatch_rows_impl(src_ptrs_host, ep_size, peer_rank, peer_token_idx, num_rows, max_rows, 0, max_rows, row_divisor,
                              hidden, dst, row_scale_ptrs_host, row_scale_out, 0, static_cast<cudaStream_t>(stream), nullptr, nullptr, nullptr);
}

extern "C" int mokb_comm_default_blocks(void) { return comm_default_blocks(); }

extern "C" int mokb_dispatch_rows_window(const uint64_t* src_ptrs_host, int ep_size, const int32_t* peer_rank,
                                         const int32_t* peer_token_idx, const int32_t* num_rows, int max_rows, int row_begin,
                                         int row_end, int row_divisor, int64_t hidden, void* dst,
                                         const uint64_t* row_scale_ptrs_host, float* row_scale_out, int blocks,
                                         int32_t* done_counter, void* q_out, void* q_sc_out, int64_t index_limit,
                                         int32_t* status, void* stream) {
    return dispatch_rows_impl(src_ptrs_host, ep_size, peer_rank, peer_token_idx, num_rows, max_rows, row_begin, row_end, row_divisor,
                              hidden, dst, row_scale_ptrs_host, row_scale_out, blocks, static_cast<cudaStream_t>(stream), done_counter,
                              q_out, q_sc_out, index_limit, status);
}

extern "C" int mokb_combine_rows(const void* src, const uint64_t* dst_ptrs_host, int ep_size,
                                 const int32_t* peer_rank, const int32_t* peer_token_idx,
                                 const int32_t* num_rows, int max_rows, int64_t hidden,
                                 const float* row_values, const uint64_t* value_ptrs_host, void* stream) {
    return combine_rows_impl(src, dst_ptrs_host, ep_size, peer_rank, peer_token_idx, num_rows, max_rows, 0, max_rows, hidden,
                             row_values, value_ptrs_host, 0, static_cast<cudaStream_t>(stream), nullptr, 0, nullptr);
}

extern "C" int mokb_combine_rows_window(const void* src, const uint64_t* dst_ptrs_host, int ep_size,
                                        const int32_t* peer_rank, const int32_t* peer_token_idx,
                                        const int32_t* num_rows, int max_rows, int row_begin, int row_end, int64_t hidden,
                                        const float* row_values, const uint64_t* value_ptrs_host, int blocks,
                                        const int32_t* wait_counter, int arrivals_per_row_block, int32_t* status,
                                        int64_t index_limit, void* stream) {
    return combine_rows_impl(src, dst_ptrs_host, ep_size, peer_rank, peer_token_idx, num_rows, max_rows, row_begin, row_end, hidden,
                             row_values, value_ptrs_host, blocks, static_cast<cudaStream_t>(stream), wait_counter,
                             arrivals_per_row_block, status, index_limit);
}
