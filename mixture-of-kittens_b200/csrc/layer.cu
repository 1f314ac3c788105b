// The fused MoE layer, forward and backward (BF16): the sequence of dispatch,
// grouped GEMMs, SwiGLU and combine that replaces the reference's persistent
// kernels (csrc/megakernel/forward.cuh:1-291, backward.cuh:1-443).
//
// Nothing here synchronises the host: the number of routed rows is read on the
// device by every kernel (forward.cuh:20 does the same).  Communication overlaps
// computation the way the reference's communication CTAs do, but with stream
// ordering instead of in-kernel counters: dispatch and combine run on two side
// streams of this library, in row windows of `minibatch_size` rows, on
// `num_comm_sms` SMs' worth of threads, and are tied to the GEMM launches on the
// caller's stream by events (fork after the prologue, join before returning):
//
//   forward   side 1: dispatch(c0) dispatch(c1) ...
//             caller: prologue | shared gate/up, shared down | gate/up(c0) down(c0) gate/up(c1) down(c1) ...
//             side 2:                                                   combine(c0)          combine(c1) ...
//   backward  side 1: scaled dispatch of d_y
//             caller: prologue | shared backward (6 launches) | routed dgrads | routed wgrads
//             side 2:                                                          combine of d_x + router grads
//
// No kernel waits on another kernel; MOKB_OVERLAP=0 puts everything on the caller's stream.
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace mokb {
namespace {

struct Scratch {
    int32_t* expert_offsets;   // [E_l + 1] row offset of each expert segment
    int32_t* shared_offsets;   // [2] = {0, T}: the shared expert as a one-group problem
    int32_t* n_rows;           // [1] validated number of routed rows (0 if it does not fit)
    int32_t* group_of_block;   // [MB / 128]
    float* w_row;              // [MB] router weight of each routed row (backward)
    float* d_w_row;            // [MB] router-weight gradient of each routed row (backward)
};

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

Scratch carve(void* base, int E_l, int MB) {
    char* p = static_cast<char*>(base);
    Scratch s;
    s.expert_offsets = reinterpret_cast<int32_t*>(p); p += align256((E_l + 1) * 4);
    s.shared_offsets = reinterpret_cast<int32_t*>(p); p += 256;
    s.n_rows = reinterpret_cast<int32_t*>(p); p += 256;
    s.group_of_block = reinterpret_cast<int32_t*>(p); p += align256(static_cast<size_t>(MB / 128) * 4);
    s.w_row = reinterpret_cast<float*>(p); p += align256(static_cast<size_t>(MB) * 4);
    s.d_w_row = reinterpret_cast<float*>(p);
    return s;
}

// One CTA: segment offsets from tokens_per_expert, row-block -> expert table,
// and the capacity checks that the reference turns into a trap.
__global__ void prologue_kernel(const int32_t* __restrict__ tokens_per_expert, const int32_t* __restrict__ num_tokens,
                                int E_l, int capacity, int MB, int T, Scratch s, int32_t* status) {
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
        else if (n > MB) { ok = 0; atomicCAS(status, MOKB_ST_OK, MOKB_ST_MACROBATCH_OVERFLOW); }
        ok_s = ok;
        *s.n_rows = ok ? n : 0;
        s.shared_offsets[0] = 0;
        s.shared_offsets[1] = T;
    }
    __syncthreads();
    const int ok = ok_s;
    for (int e = threadIdx.x; e <= E_l; e += blockDim.x) s.expert_offsets[e] = ok ? offs[e] : 0;
    const int nblocks = ok ? offs[E_l] / 128 : 0;
    for (int b = threadIdx.x; b < MB / 128; b += blockDim.x) {
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
}

int run_prologue(const int32_t* tpe, const int32_t* num_tokens, int E_l, int C, int MB, int T, const Scratch& s,
                 int32_t* status, cudaStream_t stream) {
    MOKB_REQUIRE(E_l <= 2048, "layer: at most 2048 local experts");
    prologue_kernel<<<1, 256, 0, stream>>>(tpe, num_tokens, E_l, C, MB, T, s, status);
    MOKB_CUDA(cudaGetLastError());
    note_launch();
    return MOKB_OK;
}

mokb_gemm_args gemm_base(int32_t* status) {
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

// ---- side streams and events, one set per device, created on first use
constexpr int kMaxChunks = 32;

struct Async {
    bool ready = false;
    cudaStream_t s1 = nullptr, s2 = nullptr;
    cudaEvent_t fork = nullptr, join1 = nullptr, join2 = nullptr;
    cudaEvent_t ev_in[kMaxChunks] = {nullptr};    // dispatch of chunk c finished
    cudaEvent_t ev_out[kMaxChunks] = {nullptr};   // rows of chunk c are ready to be combined
};
Async g_async[64];

int get_async(Async** out) {
    int dev = -1;
    MOKB_CUDA(cudaGetDevice(&dev));
    MOKB_REQUIRE(dev >= 0 && dev < 64, "layer: device index %d out of range", dev);
    Async& a = g_async[dev];
    if (!a.ready) {
        MOKB_CUDA(cudaStreamCreateWithFlags(&a.s1, cudaStreamNonBlocking));
        MOKB_CUDA(cudaStreamCreateWithFlags(&a.s2, cudaStreamNonBlocking));
        cudaEvent_t* single[3] = {&a.fork, &a.join1, &a.join2};
        for (auto e : single) MOKB_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        for (int c = 0; c < kMaxChunks; ++c) {
            MOKB_CUDA(cudaEventCreateWithFlags(&a.ev_in[c], cudaEventDisableTiming));
            MOKB_CUDA(cudaEventCreateWithFlags(&a.ev_out[c], cudaEventDisableTiming));
        }
        a.ready = true;
    }
    *out = &a;
    return MOKB_OK;
}

bool overlap_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MOKB_OVERLAP");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// rows per communication/compute window: minibatch_size, coarsened so that at most kMaxChunks windows cover MB
int chunk_rows_for(int MB, int minibatch) {
    int rows = minibatch;
    if ((MB + rows - 1) / rows > kMaxChunks) rows = static_cast<int>(align256((MB + kMaxChunks - 1) / kMaxChunks));
    return rows;
}

}  // namespace
}  // namespace mokb

using namespace mokb;

extern "C" size_t mokb_layer_scratch_bytes(int schedule_capacity, int num_local_experts, int macrobatch_size) {
    (void)schedule_capacity;
    return align256((num_local_experts + 1) * 4) + 512 + align256(static_cast<size_t>(macrobatch_size / 128) * 4) +
           2 * align256(static_cast<size_t>(macrobatch_size) * 4);
}

extern "C" int mokb_dispatch_mlp_swiglu_combine_fwd_bf16(const mokb_fwd_bf16_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_TRY(check_common(a, "fwd_bf16"));
    MOKB_REQUIRE(a->x_ptrs_host && a->w_shared_gate && a->w_shared_up && a->w_routed_gate && a->w_routed_up, "fwd_bf16: null input");
    MOKB_REQUIRE(a->x_routed && a->gate_shared && a->up_shared && a->hidden_shared && a->gate_routed && a->up_routed && a->hidden_routed,
                 "fwd_bf16: null output");
    const bool with_down = !a->skip_down_combine;
    if (with_down)
        MOKB_REQUIRE(a->combine_ptrs_host && a->w_shared_down && a->w_routed_down && a->y_shared && a->y_routed, "fwd_bf16: null down/combine pointer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const Scratch s = carve(a->scratch, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream, s_out = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;
    const int chunk = chunk_rows_for(MB, a->minibatch_size);
    const int nchunks = (MB + chunk - 1) / chunk;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        if (with_down) MOKB_CUDA(cudaStreamWaitEvent(s_out, as->fork, 0));
    }
    // dispatch: pull every scheduled row from its home rank, window by window
    for (int c = 0; c < nchunks; ++c) {
        const int r0 = c * chunk, r1 = r0 + chunk < MB ? r0 + chunk : MB;
        MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, r0, r1, a->topk, H,
                                    a->x_routed, nullptr, nullptr, comm_blocks, s_in));
        if (overlap) MOKB_CUDA(cudaEventRecord(as->ev_in[c], s_in));
    }
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));

    // shared expert: gate/up + SwiGLU in one pass, then down (independent of the dispatch)
    mokb_gemm_args g = gemm_base(a->status);
    g.mode = 1; g.rows_static = T; g.N = I; g.K = H;
    g.A = x_local; g.lda = H; g.B = a->w_shared_gate; g.B2 = a->w_shared_up; g.ldb = H;
    g.D = a->gate_shared; g.D2 = a->up_shared; g.D3 = a->hidden_shared; g.ldd = I;
    g.has_swiglu_limit = a->has_swiglu_limit; g.swiglu_limit = a->swiglu_limit;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    if (with_down) {
        g = gemm_base(a->status);
        g.mode = 0; g.rows_static = T; g.N = H; g.K = I;
        g.A = a->hidden_shared; g.lda = I; g.B = a->w_shared_down; g.ldb = I; g.D = a->y_shared; g.ldd = H;
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    }

    // routed experts, window by window behind the dispatch
    for (int c = 0; c < nchunks; ++c) {
        const int r0 = c * chunk, r1 = r0 + chunk < MB ? r0 + chunk : MB;
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[c], 0));
        g = gemm_base(a->status);
        g.mode = 1; g.rows_static = MB; g.row_begin = r0; g.row_end = r1;
        g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = I; g.K = H;
        g.A = a->x_routed; g.lda = H; g.B = a->w_routed_gate; g.B2 = a->w_routed_up; g.ldb = H;
        g.D = a->gate_routed; g.D2 = a->up_routed; g.D3 = a->hidden_routed; g.ldd = I;
        g.has_swiglu_limit = a->has_swiglu_limit; g.swiglu_limit = a->swiglu_limit;
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        if (!with_down) continue;
        g = gemm_base(a->status);
        g.mode = 0; g.rows_static = MB; g.row_begin = r0; g.row_end = r1;
        g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = H; g.K = I;
        g.A = a->hidden_routed; g.lda = I; g.B = a->w_routed_down; g.ldb = I; g.D = a->y_routed; g.ldd = H;
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        // combine: push the window's rows back to slot t*K+k of their home ranks
        if (overlap) {
            MOKB_CUDA(cudaEventRecord(as->ev_out[c], stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_out, as->ev_out[c], 0));
        }
        MOKB_TRY(combine_rows_impl(a->y_routed, a->combine_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, r0, r1,
                                   H, nullptr, nullptr, comm_blocks, s_out));
    }
    if (overlap && with_down) {
        MOKB_CUDA(cudaEventRecord(as->join2, s_out));
        MOKB_CUDA(cudaStreamWaitEvent(stream, as->join2, 0));
    }
    return MOKB_OK;
}

extern "C" int mokb_dispatch_mlp_swiglu_combine_bwd_bf16(const mokb_bwd_bf16_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_TRY(check_common(a, "bwd_bf16"));
    MOKB_REQUIRE(a->d_y_ptrs_host && a->d_x_routed_ptrs_host && a->router_weight_ptrs_host && a->d_router_weight_ptrs_host && a->x_ptrs_host,
                 "bwd_bf16: null pointer list");
    MOKB_REQUIRE(a->w_shared_gate && a->w_shared_up && a->w_shared_down && a->w_routed_gate && a->w_routed_up && a->w_routed_down, "bwd_bf16: null weight");
    MOKB_REQUIRE(a->x_routed && a->gate_shared && a->gate_routed && a->up_shared && a->up_routed && a->hidden_shared && a->hidden_routed,
                 "bwd_bf16: null forward context");
    MOKB_REQUIRE(a->d_x_shared && a->d_x_routed && a->d_gate_shared && a->d_gate_routed && a->d_up_shared && a->d_up_routed &&
                 a->d_hidden_shared && a->d_hidden_routed && a->d_y_routed && a->d_w_shared_gate && a->d_w_routed_gate &&
                 a->d_w_shared_up && a->d_w_routed_up && a->d_w_shared_down && a->d_w_routed_down, "bwd_bf16: null output");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const Scratch s = carve(a->scratch, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream, s_out = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;
    const int lim = a->has_swiglu_limit;
    const float limv = a->swiglu_limit;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
    }
    // reverse combine: pull d_y rows, scaled by the route's router weight (overlaps the shared expert's backward)
    MOKB_TRY(dispatch_rows_impl(a->d_y_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB, a->topk, H,
                                a->d_y_routed, a->router_weight_ptrs_host, s.w_row, comm_blocks, s_in));
    if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));
    const void* d_y_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->d_y_ptrs_host[a->ep_rank]));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));

    // ---- shared expert
    mokb_gemm_args g = gemm_base(a->status);
    g.mode = 2; g.rows_static = T; g.N = I; g.K = H;
    g.A = d_y_local; g.lda = H; g.B = a->w_shared_down; g.ldb = I; g.D = a->d_hidden_shared; g.ldd = I;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    MOKB_TRY(mokb_swiglu_bwd(a->gate_shared, a->up_shared, a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr, nullptr,
                             nullptr, T, I, lim, limv, stream));
    g = gemm_base(a->status);
    g.mode = 2; g.rows_static = T; g.N = H; g.K = I;
    g.A = a->d_gate_shared; g.B = a->w_shared_gate; g.A2 = a->d_up_shared; g.B2 = a->w_shared_up; g.lda = I; g.ldb = H;
    g.D = a->d_x_shared; g.ldd = H;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    auto wgrad = [&](const void* A, int M, const void* B, int N, void* D, int G, int rows, const int32_t* offs) -> int {
        mokb_gemm_args w = gemm_base(a->status);
        w.mode = 3; w.rows_static = rows; w.G = G; w.M = M; w.N = N; w.group_offsets = offs;
        w.A = A; w.lda = M; w.B = B; w.ldb = N; w.D = D; w.ldd = N;
        return mokb_grouped_gemm_bf16(&w, stream);
    };
    MOKB_TRY(wgrad(d_y_local, H, a->hidden_shared, I, a->d_w_shared_down, 1, T, s.shared_offsets));
    MOKB_TRY(wgrad(a->d_gate_shared, I, x_local, H, a->d_w_shared_gate, 1, T, s.shared_offsets));
    MOKB_TRY(wgrad(a->d_up_shared, I, x_local, H, a->d_w_shared_up, 1, T, s.shared_offsets));

    // ---- routed experts
    if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
    g = gemm_base(a->status);
    g.mode = 2; g.rows_static = MB; g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = I; g.K = H;
    g.A = a->d_y_routed; g.lda = H; g.B = a->w_routed_down; g.ldb = I; g.D = a->d_hidden_routed; g.ldd = I;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    MOKB_TRY(mokb_swiglu_bwd(a->gate_routed, a->up_routed, a->d_hidden_routed, a->d_gate_routed, a->d_up_routed, s.w_row, s.d_w_row,
                             s.n_rows, MB, I, lim, limv, stream));
    g = gemm_base(a->status);
    g.mode = 2; g.rows_static = MB; g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = H; g.K = I;
    g.A = a->d_gate_routed; g.B = a->w_routed_gate; g.A2 = a->d_up_routed; g.B2 = a->w_routed_up; g.lda = I; g.ldb = H;
    g.D = a->d_x_routed; g.ldd = H;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    // reverse dispatch: push d_x rows and the per-route router-weight gradient home (overlaps the weight gradients)
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->ev_out[0], stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_out, as->ev_out[0], 0));
    }
    MOKB_TRY(combine_rows_impl(a->d_x_routed, a->d_x_routed_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB,
                               H, s.d_w_row, a->d_router_weight_ptrs_host, comm_blocks, s_out));
    if (overlap) MOKB_CUDA(cudaEventRecord(as->join2, s_out));
    MOKB_TRY(wgrad(a->d_y_routed, H, a->hidden_routed, I, a->d_w_routed_down, E_l, MB, s.expert_offsets));
    MOKB_TRY(wgrad(a->d_gate_routed, I, a->x_routed, H, a->d_w_routed_gate, E_l, MB, s.expert_offsets));
    MOKB_TRY(wgrad(a->d_up_routed, I, a->x_routed, H, a->d_w_routed_up, E_l, MB, s.expert_offsets));
    if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join2, 0));
    return MOKB_OK;
}

// ============================================================================
// MXFP8: routed experts in block-scaled E4M3, shared expert in BF16
// (reference: csrc/megakernel/forward.cuh:296-428, backward.cuh:448-679).
//
// Dataflow (quantisation points as in the reference):
//   forward   dispatch x -> quantise x row-wise (GEMM operand) and token-wise (saved for wgrad)
//             gate, up = x_q * Wg_q^T, x_q * Wu_q^T (bf16) -> SwiGLU -> quantise gate, up (saved),
//             hidden row-wise (GEMM operand) and token-wise (saved) -> y = hidden_q * Wd_q^T -> combine
//   backward  pull d_y * w -> quantise both ways -> d_hidden = d_y_q * WdT_q^T
//             -> de-quantise saved gate/up, SwiGLU backward, router-gradient partials, quantise d_gate, d_up
//             both ways -> d_x = d_gate_q * WgT_q^T + d_up_q * WuT_q^T -> combine;
//             weight gradients contract the token-wise quantised tensors over each expert's rows.
// Dispatch / combine overlap the shared expert's BF16 GEMMs and the weight gradients on the side streams.
namespace mokb {
namespace {

mokb_gemm_fp8_args fp8_base(int32_t* status) {
    mokb_gemm_fp8_args g;
    memset(&g, 0, sizeof(g));
    g.G = 1;
    g.status = status;
    return g;
}

}  // namespace
}  // namespace mokb

extern "C" int mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8(const mokb_fwd_mxfp8_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_TRY(check_common(a, "fwd_mxfp8"));
    MOKB_REQUIRE(a->intermediate % 128 == 0 && a->hidden % 128 == 0, "fwd_mxfp8: hidden and intermediate must be multiples of 128");
    MOKB_REQUIRE(a->x_ptrs_host && a->w_shared_gate && a->w_shared_up && a->w_routed_gate && a->w_routed_gate_sc && a->w_routed_up &&
                 a->w_routed_up_sc, "fwd_mxfp8: null input");
    MOKB_REQUIRE(a->x_fp8_t && a->x_sc_t && a->gate_shared && a->up_shared && a->hidden_shared && a->gate_fp8 && a->gate_sc &&
                 a->up_fp8 && a->up_sc && a->hidden_fp8_t && a->hidden_sc_t, "fwd_mxfp8: null output");
    MOKB_REQUIRE(a->x_routed && a->x_fp8 && a->x_sc && a->gate_bf16 && a->up_bf16 && a->hidden_fp8 && a->hidden_sc, "fwd_mxfp8: null work buffer");
    const bool with_down = !a->skip_down_combine;
    if (with_down)
        MOKB_REQUIRE(a->combine_ptrs_host && a->w_shared_down && a->w_routed_down && a->w_routed_down_sc && a->y_shared && a->y_routed,
                     "fwd_mxfp8: null down/combine pointer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const Scratch s = carve(a->scratch, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
    }
    // dispatch + quantise (row-wise for the GEMM, token-wise for the weight gradients) on the side stream
    MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB, a->topk, H,
                                a->x_routed, nullptr, nullptr, comm_blocks, s_in));
    MOKB_TRY(quantize_impl(a->x_routed, 1, MB, H, s.n_rows, a->x_fp8, a->x_sc, a->x_fp8_t, a->x_sc_t, s_in));
    if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));

    // shared expert (BF16)
    mokb_gemm_args g = gemm_base(a->status);
    g.mode = 1; g.rows_static = T; g.N = I; g.K = H;
    g.A = x_local; g.lda = H; g.B = a->w_shared_gate; g.B2 = a->w_shared_up; g.ldb = H;
    g.D = a->gate_shared; g.D2 = a->up_shared; g.D3 = a->hidden_shared; g.ldd = I;
    g.has_swiglu_limit = a->has_swiglu_limit; g.swiglu_limit = a->swiglu_limit;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    if (with_down) {
        g = gemm_base(a->status);
        g.mode = 0; g.rows_static = T; g.N = H; g.K = I;
        g.A = a->hidden_shared; g.lda = I; g.B = a->w_shared_down; g.ldb = I; g.D = a->y_shared; g.ldd = H;
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    }

    // routed experts (MXFP8)
    if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
    mokb_gemm_fp8_args f = fp8_base(a->status);
    f.mode = 1; f.rows_static = MB; f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
    f.A = a->x_fp8; f.A_sc = a->x_sc; f.B = a->w_routed_gate; f.B_sc = a->w_routed_gate_sc; f.B2 = a->w_routed_up; f.B2_sc = a->w_routed_up_sc;
    f.D = a->gate_bf16; f.D2 = a->up_bf16; f.ldd = I;
    MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
    MOKB_TRY(swiglu_fwd_quant_impl(a->gate_bf16, a->up_bf16, MB, I, s.n_rows, a->has_swiglu_limit, a->swiglu_limit, a->gate_fp8, a->gate_sc,
                                   a->up_fp8, a->up_sc, a->hidden_fp8, a->hidden_sc, a->hidden_fp8_t, a->hidden_sc_t, stream));
    if (with_down) {
        f = fp8_base(a->status);
        f.mode = 0; f.rows_static = MB; f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = H; f.K = I;
        f.A = a->hidden_fp8; f.A_sc = a->hidden_sc; f.B = a->w_routed_down; f.B_sc = a->w_routed_down_sc; f.D = a->y_routed; f.ldd = H;
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        MOKB_TRY(combine_rows_impl(a->y_routed, a->combine_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB, H,
                                   nullptr, nullptr, 0, stream));
    }
    return MOKB_OK;
}

extern "C" int mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8(const mokb_bwd_mxfp8_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_TRY(check_common(a, "bwd_mxfp8"));
    MOKB_REQUIRE(a->d_y_ptrs_host && a->d_x_routed_ptrs_host && a->router_weight_ptrs_host && a->d_router_weight_ptrs_host && a->x_ptrs_host,
                 "bwd_mxfp8: null pointer list");
    MOKB_REQUIRE(a->w_shared_gate && a->w_shared_up && a->w_shared_down && a->w_routed_gate_t && a->w_routed_gate_t_sc && a->w_routed_up_t &&
                 a->w_routed_up_t_sc && a->w_routed_down_t && a->w_routed_down_t_sc, "bwd_mxfp8: null weight");
    MOKB_REQUIRE(a->x_fp8_t && a->x_sc_t && a->gate_shared && a->gate_fp8 && a->gate_sc && a->up_shared && a->up_fp8 && a->up_sc &&
                 a->hidden_shared && a->hidden_fp8_t && a->hidden_sc_t, "bwd_mxfp8: null forward context");
    MOKB_REQUIRE(a->d_x_shared && a->d_x_routed && a->d_gate_shared && a->d_gate_fp8 && a->d_gate_sc && a->d_up_shared && a->d_up_fp8 &&
                 a->d_up_sc && a->d_hidden_shared && a->d_hidden_routed && a->d_y_fp8 && a->d_y_sc && a->d_w_shared_gate &&
                 a->d_w_routed_gate && a->d_w_shared_up && a->d_w_routed_up && a->d_w_shared_down && a->d_w_routed_down, "bwd_mxfp8: null output");
    MOKB_REQUIRE(a->d_y_routed && a->d_y_fp8_t && a->d_y_sc_t && a->d_gate_fp8_t && a->d_gate_sc_t && a->d_up_fp8_t && a->d_up_sc_t && a->partials,
                 "bwd_mxfp8: null work buffer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const Scratch s = carve(a->scratch, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream, s_out = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;
    const int lim = a->has_swiglu_limit;
    const float limv = a->swiglu_limit;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
    }
    MOKB_TRY(dispatch_rows_impl(a->d_y_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB, a->topk, H,
                                a->d_y_routed, a->router_weight_ptrs_host, s.w_row, comm_blocks, s_in));
    MOKB_TRY(quantize_impl(a->d_y_routed, 1, MB, H, s.n_rows, a->d_y_fp8, a->d_y_sc, a->d_y_fp8_t, a->d_y_sc_t, s_in));
    if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));
    const void* d_y_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->d_y_ptrs_host[a->ep_rank]));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));

    // ---- shared expert (BF16)
    mokb_gemm_args g = gemm_base(a->status);
    g.mode = 2; g.rows_static = T; g.N = I; g.K = H;
    g.A = d_y_local; g.lda = H; g.B = a->w_shared_down; g.ldb = I; g.D = a->d_hidden_shared; g.ldd = I;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    MOKB_TRY(mokb_swiglu_bwd(a->gate_shared, a->up_shared, a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr, nullptr,
                             nullptr, T, I, lim, limv, stream));
    g = gemm_base(a->status);
    g.mode = 2; g.rows_static = T; g.N = H; g.K = I;
    g.A = a->d_gate_shared; g.B = a->w_shared_gate; g.A2 = a->d_up_shared; g.B2 = a->w_shared_up; g.lda = I; g.ldb = H;
    g.D = a->d_x_shared; g.ldd = H;
    MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
    auto wgrad_bf16 = [&](const void* A, int M, const void* B, int N, void* D) -> int {
        mokb_gemm_args w = gemm_base(a->status);
        w.mode = 3; w.rows_static = T; w.G = 1; w.M = M; w.N = N; w.group_offsets = s.shared_offsets;
        w.A = A; w.lda = M; w.B = B; w.ldb = N; w.D = D; w.ldd = N;
        return mokb_grouped_gemm_bf16(&w, stream);
    };
    MOKB_TRY(wgrad_bf16(d_y_local, H, a->hidden_shared, I, a->d_w_shared_down));
    MOKB_TRY(wgrad_bf16(a->d_gate_shared, I, x_local, H, a->d_w_shared_gate));
    MOKB_TRY(wgrad_bf16(a->d_up_shared, I, x_local, H, a->d_w_shared_up));

    // ---- routed experts (MXFP8)
    if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
    mokb_gemm_fp8_args f = fp8_base(a->status);
    f.mode = 0; f.rows_static = MB; f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
    f.A = a->d_y_fp8; f.A_sc = a->d_y_sc; f.B = a->w_routed_down_t; f.B_sc = a->w_routed_down_t_sc; f.D = a->d_hidden_routed; f.ldd = I;
    MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
    MOKB_TRY(swiglu_bwd_quant_impl(a->gate_fp8, a->gate_sc, a->up_fp8, a->up_sc, a->d_hidden_routed, MB, I, s.n_rows, lim, limv, s.w_row,
                                   a->d_gate_fp8, a->d_gate_sc, a->d_gate_fp8_t, a->d_gate_sc_t, a->d_up_fp8, a->d_up_sc, a->d_up_fp8_t,
                                   a->d_up_sc_t, static_cast<float*>(a->partials), s.d_w_row, stream));
    f = fp8_base(a->status);
    f.mode = 0; f.rows_static = MB; f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = H; f.K = I;
    f.A = a->d_gate_fp8; f.A_sc = a->d_gate_sc; f.B = a->w_routed_gate_t; f.B_sc = a->w_routed_gate_t_sc;
    f.A2 = a->d_up_fp8; f.A2_sc = a->d_up_sc; f.B2 = a->w_routed_up_t; f.B2_sc = a->w_routed_up_t_sc; f.D = a->d_x_routed; f.ldd = H;
    MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->ev_out[0], stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_out, as->ev_out[0], 0));
    }
    MOKB_TRY(combine_rows_impl(a->d_x_routed, a->d_x_routed_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB,
                               H, s.d_w_row, a->d_router_weight_ptrs_host, comm_blocks, s_out));
    if (overlap) MOKB_CUDA(cudaEventRecord(as->join2, s_out));
    auto wgrad_fp8 = [&](const void* A, const void* A_sc, int M, const void* B, const void* B_sc, int N, void* D) -> int {
        mokb_gemm_fp8_args w = fp8_base(a->status);
        w.mode = 2; w.rows_static = MB; w.G = E_l; w.M = M; w.N = N; w.group_offsets = s.expert_offsets;
        w.A = A; w.A_sc = A_sc; w.B = B; w.B_sc = B_sc; w.D = D; w.ldd = N;
        return mokb_grouped_gemm_mxfp8(&w, stream);
    };
    MOKB_TRY(wgrad_fp8(a->d_y_fp8_t, a->d_y_sc_t, H, a->hidden_fp8_t, a->hidden_sc_t, I, a->d_w_routed_down));
    MOKB_TRY(wgrad_fp8(a->d_gate_fp8_t, a->d_gate_sc_t, I, a->x_fp8_t, a->x_sc_t, H, a->d_w_routed_gate));
    MOKB_TRY(wgrad_fp8(a->d_up_fp8_t, a->d_up_sc_t, I, a->x_fp8_t, a->x_sc_t, H, a->d_w_routed_up));
    if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join2, 0));
    return MOKB_OK;
}
