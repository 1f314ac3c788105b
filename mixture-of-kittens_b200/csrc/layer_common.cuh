// Pieces shared by the BF16 and MXFP8 layer launchers: the scratch layout, the prologue kernel
// that turns tokens_per_expert into the tables the GEMMs read, and the side streams / events
// used to overlap dispatch and combine with the GEMMs.
#pragma once

#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace mokb {
namespace {

// Routed rows are processed in macrobatches of MB rows (the reference's ring buffer,
// csrc/megakernel/types.cuh:86-106): macrobatch m owns schedule rows [m*MB, (m+1)*MB) and every
// [MB, .] buffer holds row r of macrobatch m at r - m*MB.
struct Scratch {
    int32_t* expert_offsets;   // [E_l + 1] row offset of each expert segment
    int32_t* shared_offsets;   // [2] = {0, T}: the shared expert as a one-group problem
    int32_t* n_rows;           // [1] validated number of routed rows (0 if the schedule is unusable)
    int32_t* mb_rows;          // [n_macro] rows of macrobatch m
    int32_t* mb_offsets;       // [n_macro][E_l + 1] expert offsets clamped to macrobatch m's row range
    int32_t* mb_k_end;         // [n_macro][E_l] end of each expert's scheduled rows (the rest of its segment is padding), clamped likewise
    int32_t* group_of_block;   // [capacity / 128]
    float* w_row;              // [MB] router weight of each routed row of the current macrobatch (backward)
    float* d_w_row;            // [MB] router-weight gradient of each routed row (backward)
    // counters between kernels that run at the same time (zeroed by the prologue of every call)
    int32_t* win_ready;        // [kMaxChunks] blocks of the dispatch launch of window w that have finished
    int32_t* win_done;         // [kMaxChunks] epilogue warps that have stored a down tile of window w
    int32_t* blk_done;         // [capacity / 256] epilogue warps that have stored a gate/up tile of a 256-row block
};

inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

inline int macrobatches(int capacity, int MB) { return (capacity + MB - 1) / MB; }

constexpr int kMaxChunks = 32;     // windows per macrobatch (side-stream events, counters)
// `num_comm_sms` SMs' worth of communication threads: 2048 per SM, in blocks of 128 (see comm.cu)
constexpr int kCommBlocksPerSm = 16;

inline size_t scratch_bytes(int capacity, int E_l, int MB) {
    const size_t nm = macrobatches(capacity, MB);
    return align256((E_l + 1) * 4) + 512 + align256(nm * 4) + 2 * align256(nm * (E_l + 1) * 4) +
           align256(static_cast<size_t>(capacity / 128) * 4) + 2 * align256(static_cast<size_t>(MB) * 4) +
           2 * align256(kMaxChunks * 4) + align256(static_cast<size_t>(capacity / 256) * 4);
}

inline Scratch carve(void* base, int capacity, int E_l, int MB) {
    const size_t nm = macrobatches(capacity, MB);
    char* p = static_cast<char*>(base);
    Scratch s;
    s.expert_offsets = reinterpret_cast<int32_t*>(p); p += align256((E_l + 1) * 4);
    s.shared_offsets = reinterpret_cast<int32_t*>(p); p += 256;
    s.n_rows = reinterpret_cast<int32_t*>(p); p += 256;
    s.mb_rows = reinterpret_cast<int32_t*>(p); p += align256(nm * 4);
    s.mb_offsets = reinterpret_cast<int32_t*>(p); p += align256(nm * (E_l + 1) * 4);
    s.mb_k_end = reinterpret_cast<int32_t*>(p); p += align256(nm * (E_l + 1) * 4);
    s.group_of_block = reinterpret_cast<int32_t*>(p); p += align256(static_cast<size_t>(capacity / 128) * 4);
    s.w_row = reinterpret_cast<float*>(p); p += align256(static_cast<size_t>(MB) * 4);
    s.d_w_row = reinterpret_cast<float*>(p); p += align256(static_cast<size_t>(MB) * 4);
    s.win_ready = reinterpret_cast<int32_t*>(p); p += align256(kMaxChunks * 4);
    s.win_done = reinterpret_cast<int32_t*>(p); p += align256(kMaxChunks * 4);
    s.blk_done = reinterpret_cast<int32_t*>(p);
    return s;
}

// One CTA: segment offsets from tokens_per_expert, row-block -> expert table, per-macrobatch
// offsets, and the capacity check that the reference turns into a trap.
__global__ void prologue_kernel(const int32_t* __restrict__ tokens_per_expert, const int32_t* __restrict__ num_tokens,
                                const int32_t* __restrict__ peer_rank, int E_l, int capacity, int MB, int T, Scratch s, int32_t* status) {
    __shared__ int32_t offs[2049];
    __shared__ int32_t ok_s;
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E_l; ++e) {
            offs[e] = run;
            run += tokens_per_expert[e];
        }
        offs[E_l] = run;
        const int n = *num_tokens;
        int ok = 1;
        if (n != run || n < 0 || n > capacity) { ok = 0; atomicCAS(status, MOKB_ST_OK, MOKB_ST_SCHEDULE_OVERFLOW); }
        ok_s = ok;
        *s.n_rows = ok ? n : 0;
        s.shared_offsets[0] = 0;
        s.shared_offsets[1] = T;
    }
    __syncthreads();
    const int ok = ok_s;
    const int total = ok ? offs[E_l] : 0;
    for (int e = threadIdx.x; e <= E_l; e += blockDim.x) s.expert_offsets[e] = ok ? offs[e] : 0;
    const int nm = (capacity + MB - 1) / MB;
    for (int e = threadIdx.x; e < E_l; e += blockDim.x) {
        // the scheduled rows of an expert come first in its segment and fewer than 256 padding rows follow
        // (csrc/scheduler.cuh:134-139): find where the padding starts in the segment's last 256 rows
        int end = ok ? offs[e + 1] : 0;
        const int begin = ok ? offs[e] : 0;
        if (end > begin) {
            int lo = end - 256, hi = end;          // first row in [lo, hi) with peer_rank < 0, or hi
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (peer_rank[mid] < 0) hi = mid; else lo = mid + 1;
            }
            end = lo;
        }
        for (int m = 0; m < nm; ++m) s.mb_k_end[m * (E_l + 1) + e] = min(max(end, m * MB), m * MB + MB);
    }
    for (int m = 0; m < nm; ++m) {
        const int lo = m * MB, hi = lo + MB;
        for (int e = threadIdx.x; e <= E_l; e += blockDim.x) {
            const int o = ok ? offs[e] : 0;
            s.mb_offsets[m * (E_l + 1) + e] = min(max(o, lo), hi);
        }
        if (threadIdx.x == 0) s.mb_rows[m] = min(max(total - lo, 0), MB);
    }
    const int nblocks = total / 128;
    for (int b = threadIdx.x; b < capacity / 128; b += blockDim.x) {
        int g = -1;
        if (b < nblocks) {
            const int row = b * 128;
            int lo = 0, hi = E_l;          // last e with offs[e] <= row
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offs[mid] <= row) lo = mid; else hi = mid;
            }
            g = lo;
        }
        s.group_of_block[b] = g;
    }
    for (int i = threadIdx.x; i < kMaxChunks; i += blockDim.x) s.win_ready[i] = s.win_done[i] = 0;
    for (int i = threadIdx.x; i < capacity / 256; i += blockDim.x) s.blk_done[i] = 0;
}

inline int run_prologue(const int32_t* tpe, const int32_t* num_tokens, const int32_t* peer_rank, int E_l, int C, int MB, int T, const Scratch& s,
                        int32_t* status, cudaStream_t stream) {
    MOKB_REQUIRE(E_l <= 2048, "layer: at most 2048 local experts");
    prologue_kernel<<<1, 256, 0, stream>>>(tpe, num_tokens, peer_rank, E_l, C, MB, T, s, status);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

inline mokb_gemm_args gemm_base(int32_t* status) {
    mokb_gemm_args g;
    memset(&g, 0, sizeof(g));
    g.G = 1;
    g.status = status;
    return g;
}

template <class A>
int check_common(const A* a, const char* who) {
    MOKB_REQUIRE(a != nullptr, "%s: null args", who);
    MOKB_REQUIRE(a->ep_size >= 1 && a->ep_size <= MOKB_MAX_EP && a->ep_rank >= 0 && a->ep_rank < a->ep_size, "%s: bad ep_size/ep_rank", who);
    MOKB_REQUIRE(a->num_local_tokens > 0 && a->num_local_tokens % 256 == 0, "%s: num_local_tokens must be a positive multiple of 256", who);
    MOKB_REQUIRE(a->hidden > 0 && a->hidden % 256 == 0, "%s: hidden must be a positive multiple of 256", who);
    MOKB_REQUIRE(a->intermediate > 0 && a->intermediate % 128 == 0, "%s: intermediate must be a positive multiple of 128", who);
    MOKB_REQUIRE(a->num_local_experts > 0 && a->topk > 0 && a->topk <= 255, "%s: bad expert/top-k counts", who);
    MOKB_REQUIRE(a->schedule_capacity > 0 && a->schedule_capacity % 256 == 0, "%s: schedule_capacity must be a positive multiple of 256", who);
    MOKB_REQUIRE(a->macrobatch_size > 0 && a->macrobatch_size % 256 == 0, "%s: macrobatch_size must be a positive multiple of 256", who);
    MOKB_REQUIRE(a->minibatch_size > 0 && a->minibatch_size % 256 == 0, "%s: minibatch_size must be a positive multiple of 256", who);
    MOKB_REQUIRE(a->num_comm_sms > 0, "%s: num_comm_sms must be positive", who);
    MOKB_REQUIRE(a->peer_rank && a->peer_token_idx && a->num_tokens && a->tokens_per_expert, "%s: null schedule pointer", who);
    MOKB_REQUIRE(a->scratch && a->status, "%s: scratch and status are required", who);
    return MOKB_OK;
}

}  // namespace

// ---- side streams and events, one set per device, created on first use (defined in layer.cu)

struct Async {
    bool ready = false;
    cudaStream_t s1 = nullptr, s2 = nullptr;
    cudaEvent_t fork = nullptr, join1 = nullptr, join2 = nullptr;
    cudaEvent_t ev_in[kMaxChunks] = {nullptr};    // dispatch of window c finished
    cudaEvent_t ev_out[kMaxChunks] = {nullptr};   // rows of window c are ready to be combined
};

int get_async(Async** out);      // layer.cu
bool overlap_enabled();          // layer.cu

namespace {

// rows per communication/compute window: minibatch_size, coarsened so that at most kMaxChunks windows cover MB
inline int chunk_rows_for(int MB, int minibatch) {
    int rows = minibatch;
    if ((MB + rows - 1) / rows > kMaxChunks) rows = static_cast<int>(align256((MB + kMaxChunks - 1) / kMaxChunks));
    return rows;
}

// The backward pulls d_y in a few large windows, so that the first routed GEMM can start on the rows that have
// arrived while the rest is still in flight (macrobatch 0 only; later macrobatches are replays of small remainders).
constexpr int kBwdWindows = 4;
inline int bwd_chunk_rows(int rows, bool windowed) {
    if (!windowed || rows <= 0) return rows > 0 ? rows : 256;
    return static_cast<int>(align256((rows + kBwdWindows - 1) / kBwdWindows));
}

// Address such that element [row][0] of a [.., ld] buffer holding macrobatch rows from `first_row` on is
// reached with the schedule's own row index: buffer row = row - first_row.
template <class T>
inline T* rebase(T* buffer, int first_row, size_t row_bytes) {
    return reinterpret_cast<T*>(reinterpret_cast<uintptr_t>(buffer) - static_cast<size_t>(first_row) * row_bytes);
}

}  // namespace
}  // namespace mokb
