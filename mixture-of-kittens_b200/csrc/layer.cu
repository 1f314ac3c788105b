// The fused MoE layer, forward and backward (BF16): dispatch, grouped GEMMs, SwiGLU and combine, the work of
// the reference's persistent kernels (csrc/megakernel/forward.cuh:1-291, backward.cuh:1-443).
//
// Nothing here synchronises the host: the number of routed rows is read on the device by every kernel
// (forward.cuh:20 does the same).
//
//   forward   side stream: dispatch(w0) dispatch(w1) ...                      each raises win_ready[w] when its rows have landed
//             caller     : prologue | shared gate/up, shared down | ONE routed launch: for every window w
//                          { wait win_ready[w]; gate/up + SwiGLU tiles; down tiles, each after the gate/up tiles of its
//                            256 rows (blk_done); the down epilogue stores every row into its home rank's combine buffer }
//   backward  side stream: scaled dispatch of d_y in four windows, raising win_ready[w]
//             caller     : prologue | shared backward (6 launches) | d_hidden = d_y * W_down (one launch, window by window)
//                          | SwiGLU backward | d_x = d_gate * W_gate + d_up * W_up, whose epilogue stores every row and its
//                            router-weight gradient into the home rank's buffers | three weight gradients
//
// The counters are the reference's (csrc/megakernel/utils.cuh:1-13, types.cuh:126-130): global-memory words added to
// with release semantics by whoever produced some rows and polled with acquire loads by whoever consumes them.  Who may
// wait is restricted so that nothing can starve: only CTAs of the persistent GEMM wait, either for dispatch blocks (which
// never wait and therefore always finish) or for other CTAs of the same GEMM, whose tiles come earlier in the one order
// that every CTA walks; kernels that run beside the GEMM never wait for it, because blocks that sit on an SM waiting
// would keep the GEMM's own CTAs (one per SM, nearly all of its shared memory and a third of its registers) from
// being placed.  Every wait is bounded (2 s, then MOKB_ST_FLAG_TIMEOUT and the kernel drains and exits).
//
// Macrobatches (csrc/megakernel/types.cuh:86-106, forward.cuh:89-131, backward.cuh:286-329 of the
// reference): the routed buffers hold `macrobatch_size` rows; when the schedule has more, the rows
// are processed MB at a time.  The forward walks the macrobatches from the last to the first, so
// that macrobatch 0's intermediates are what stays saved; the backward consumes the saved context
// for macrobatch 0, and for every later one replays dispatch + gate/up + SwiGLU first.  Weight
// gradients of later macrobatches are added to the stored bf16 gradient in macrobatch order, which
// keeps results bit-reproducible.  How many macrobatches are non-empty is only known on the
// device: all ceil(capacity / MB) are enqueued and the empty ones find no rows.  Only macrobatch 0 is cut into
// windows; later ones are ordered by events.  MOKB_OVERLAP=0 puts everything on the caller's stream.
#include "layer_common.cuh"

namespace mokb {

static Async g_async[64];

int get_async(Async** out) {
    int dev = -1;
    MOKB_CUDA(cudaGetDevice(&dev));
    MOKB_REQUIRE(dev >= 0 && dev < 64, "layer: device index %d out of range", dev);
    Async& a = g_async[dev];
    if (!a.ready) {
        // s1 carries the pulls a waiting GEMM depends on, s2 work that is only needed later (the token-wise MXFP8 copies):
        // where both have blocks ready for the same free slot of an SM, the pull goes first
        int prio_low = 0, prio_high = 0;
        MOKB_CUDA(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
        MOKB_CUDA(cudaStreamCreateWithPriority(&a.s1, cudaStreamNonBlocking, prio_high));
        MOKB_CUDA(cudaStreamCreateWithPriority(&a.s2, cudaStreamNonBlocking, prio_low));
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

}  // namespace mokb

using namespace mokb;

extern "C" size_t mokb_layer_scratch_bytes(int schedule_capacity, int num_local_experts, int macrobatch_size) {
    return scratch_bytes(schedule_capacity, num_local_experts, macrobatch_size);
}

extern "C" int mokb_dispatch_mlp_swiglu_combine_fwd_bf16(const mokb_fwd_bf16_args* a, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MOKB_TRY(check_common(a, "fwd_bf16"));
    MOKB_REQUIRE(a->x_ptrs_host && a->w_shared_gate && a->w_shared_up && a->w_routed_gate && a->w_routed_up, "fwd_bf16: null input");
    MOKB_REQUIRE(a->x_routed && a->gate_shared && a->up_shared && a->hidden_shared && a->gate_routed && a->up_routed && a->hidden_routed,
                 "fwd_bf16: null output");
    const bool with_down = !a->skip_down_combine;
    if (with_down)
        MOKB_REQUIRE(a->combine_ptrs_host && a->w_shared_down && a->w_routed_down && a->y_shared, "fwd_bf16: null down/combine pointer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const int C = a->schedule_capacity;
    const int64_t routes = static_cast<int64_t>(T) * a->topk;      // every rank's routes are numbered [0, routes)
    const Scratch s = carve(a->scratch, C, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * kCommBlocksPerSm : 0;
    // recompute only rebuilds macrobatch 0 (the saved context); the forward walks all of them, last first
    const int n_macro = with_down ? macrobatches(C, MB) : 1;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, a->peer_rank, E_l, C, MB, T, s, a->status, stream));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));
    bool shared_done = false;

    for (int mi = 0; mi < n_macro; ++mi) {
        const int m = n_macro - 1 - mi;
        const int lo = m * MB, hi = (lo + MB < C) ? lo + MB : C;
        // only macrobatch 0 (the one that is always populated) is cut into overlap windows
        const int chunk = m == 0 ? chunk_rows_for(MB, a->minibatch_size) : MB;
        const int nchunks = (hi - lo + chunk - 1) / chunk;
        // windows of macrobatch 0 are tied to the GEMM launch by counters: the GEMM is ONE persistent launch that
        // starts window w when the dispatch blocks of w have arrived
        const bool flags = overlap && m == 0;
        void* x_routed = rebase(a->x_routed, lo, 2ull * H);
        void* gate_r = rebase(a->gate_routed, lo, 2ull * I);
        void* up_r = rebase(a->up_routed, lo, 2ull * I);
        void* hidden_r = rebase(a->hidden_routed, lo, 2ull * I);
        void* y_r = (with_down && a->y_routed) ? rebase(a->y_routed, lo, 2ull * H) : nullptr;

        if (overlap) {     // everything enqueued so far (previous macrobatch included) precedes this one's side work
            MOKB_CUDA(cudaEventRecord(as->fork, stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        }
        // dispatch: pull every scheduled row from its home rank, window by window
        for (int c = 0; c < nchunks; ++c) {
            const int r0 = lo + c * chunk, r1 = r0 + chunk < hi ? r0 + chunk : hi;
            MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, r0, r1, a->topk, H,
                                        x_routed, nullptr, nullptr, comm_blocks, s_in, flags ? s.win_ready + c : nullptr, nullptr, nullptr, routes, a->status));
        }
        if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));

        if (!shared_done) {
            // shared expert: gate/up + SwiGLU in one pass, then down (independent of the dispatch)
            shared_done = true;
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
        }

        // routed experts: gate/up + SwiGLU and the down projection of every window in one launch
        if (overlap && !flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
        mokb_gemm_args g = gemm_base(a->status);
        g.mode = 4; g.rows_static = hi; g.row_begin = lo; g.row_end = hi;
        g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = I; g.K = H;
        g.A = x_routed; g.lda = H; g.B = a->w_routed_gate; g.B2 = a->w_routed_up; g.ldb = H;
        g.D = gate_r; g.D2 = up_r; g.D3 = hidden_r; g.ldd = I;
        g.has_swiglu_limit = a->has_swiglu_limit; g.swiglu_limit = a->swiglu_limit;
        g.window_rows = chunk;
        g.blk_done = s.blk_done + lo / 256;
        if (flags) { g.win_ready = s.win_ready; g.win_ready_target = comm_blocks; }
        if (with_down) {
            // combine: the epilogue of every down tile stores its rows straight into slot t*K+k of their home ranks'
            // combine buffers (y_routed, when the caller wants it, gets a copy)
            g.B3 = a->w_routed_down; g.ldb3 = I; g.D4 = y_r; g.ldd4 = H; g.N2 = H;
            g.push_ptrs_host = a->combine_ptrs_host; g.push_ep_size = a->ep_size;
            g.push_rank = a->peer_rank; g.push_idx = a->peer_token_idx; g.push_index_limit = routes;
        }
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        // the next macrobatch (or the caller) reuses x_routed: the side stream must be done with it
        if (flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
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
    MOKB_REQUIRE(a->d_x_shared && a->d_gate_shared && a->d_gate_routed && a->d_up_shared && a->d_up_routed &&
                 a->d_hidden_shared && a->d_hidden_routed && a->d_y_routed && a->d_w_shared_gate && a->d_w_routed_gate &&
                 a->d_w_shared_up && a->d_w_routed_up && a->d_w_shared_down && a->d_w_routed_down, "bwd_bf16: null output");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const int C = a->schedule_capacity;
    const int64_t routes = static_cast<int64_t>(T) * a->topk;      // every rank's routes are numbered [0, routes)
    const Scratch s = carve(a->scratch, C, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * kCommBlocksPerSm : 0;
    const int lim = a->has_swiglu_limit;
    const float limv = a->swiglu_limit;
    const int n_macro = macrobatches(C, MB);

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, a->peer_rank, E_l, C, MB, T, s, a->status, stream));
    const void* d_y_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->d_y_ptrs_host[a->ep_rank]));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));
    auto wgrad = [&](const void* A, int M, const void* B, int N, void* D, int G, int rows, const int32_t* offs, int accumulate,
                     const int32_t* k_end = nullptr) -> int {
        mokb_gemm_args w = gemm_base(a->status);
        w.mode = 3; w.rows_static = rows; w.G = G; w.M = M; w.N = N; w.group_offsets = offs; w.accumulate = accumulate;
        w.group_k_end = k_end;       // the padding rows at the end of every expert's segment are zero: not multiplied
        w.A = A; w.lda = M; w.B = B; w.ldb = N; w.D = D; w.ldd = N;
        return mokb_grouped_gemm_bf16(&w, stream);
    };

    for (int m = 0; m < n_macro; ++m) {
        const int lo = m * MB, hi = (lo + MB < C) ? lo + MB : C;
        // the saved context and the routed work buffers, addressed by schedule row
        void* x_routed = rebase(const_cast<void*>(a->x_routed), lo, 2ull * H);
        void* gate_r = rebase(const_cast<void*>(a->gate_routed), lo, 2ull * I);
        void* up_r = rebase(const_cast<void*>(a->up_routed), lo, 2ull * I);
        void* hidden_r = rebase(const_cast<void*>(a->hidden_routed), lo, 2ull * I);
        void* d_y_r = rebase(a->d_y_routed, lo, 2ull * H);
        void* d_hidden_r = rebase(a->d_hidden_routed, lo, 2ull * I);
        void* d_gate_r = rebase(a->d_gate_routed, lo, 2ull * I);
        void* d_up_r = rebase(a->d_up_routed, lo, 2ull * I);
        void* d_x_r = a->d_x_routed ? rebase(a->d_x_routed, lo, 2ull * H) : nullptr;
        float* w_row = rebase(s.w_row, lo, 4);
        float* d_w_row = rebase(s.d_w_row, lo, 4);

        if (overlap) {     // the previous macrobatch's weight gradients still read the buffers the dispatches below overwrite
            MOKB_CUDA(cudaEventRecord(as->fork, stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        }
        // replay (later macrobatches only): pull x again; the saved context holds macrobatch 0
        if (m > 0)
            MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, lo, hi, a->topk, H,
                                        x_routed, nullptr, nullptr, comm_blocks, s_in, nullptr, nullptr, nullptr, routes, a->status));
        if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));     // the replayed x is in place
        // reverse combine: pull d_y rows, scaled by the route's router weight, in a few windows; in macrobatch 0 the
        // first routed GEMM is one launch that starts each window when the window's dispatch blocks have arrived
        const bool flags = overlap && m == 0;
        const int bchunk = bwd_chunk_rows(hi - lo, m == 0);
        const int nb = (hi - lo + bchunk - 1) / bchunk;
        for (int c = 0; c < nb; ++c) {
            const int r0 = lo + c * bchunk, r1 = r0 + bchunk < hi ? r0 + bchunk : hi;
            MOKB_TRY(dispatch_rows_impl(a->d_y_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, r0, r1, a->topk, H,
                                        d_y_r, a->router_weight_ptrs_host, w_row, comm_blocks, s_in, flags ? s.win_ready + c : nullptr, nullptr, nullptr,
                                        routes, a->status));
        }
        if (overlap) MOKB_CUDA(cudaEventRecord(as->ev_in[0], s_in));

        if (m == 0) {
            // ---- shared expert (overlaps the dispatch above)
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
            MOKB_TRY(wgrad(d_y_local, H, a->hidden_shared, I, a->d_w_shared_down, 1, T, s.shared_offsets, 0));
            MOKB_TRY(wgrad(a->d_gate_shared, I, x_local, H, a->d_w_shared_gate, 1, T, s.shared_offsets, 0));
            MOKB_TRY(wgrad(a->d_up_shared, I, x_local, H, a->d_w_shared_up, 1, T, s.shared_offsets, 0));
        }

        // ---- routed experts of this macrobatch
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
        mokb_gemm_args g;
        if (m > 0) {       // replay gate/up + SwiGLU into the context buffers
            g = gemm_base(a->status);
            g.mode = 1; g.rows_static = hi; g.row_begin = lo; g.row_end = hi;
            g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = I; g.K = H;
            g.A = x_routed; g.lda = H; g.B = a->w_routed_gate; g.B2 = a->w_routed_up; g.ldb = H;
            g.D = gate_r; g.D2 = up_r; g.D3 = hidden_r; g.ldd = I;
            g.has_swiglu_limit = lim; g.swiglu_limit = limv;
            MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        }
        // d_hidden = d_y * W_down, window by window behind the pull
        if (overlap && !flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[0], 0));
        g = gemm_base(a->status);
        g.mode = 2; g.rows_static = hi; g.row_begin = lo; g.row_end = hi;
        g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = I; g.K = H;
        g.A = d_y_r; g.lda = H; g.B = a->w_routed_down; g.ldb = I; g.D = d_hidden_r; g.ldd = I;
        if (flags) { g.window_rows = bchunk; g.win_ready = s.win_ready; g.win_ready_target = comm_blocks; }
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        // (the pulls have all arrived once that GEMM is through its last window; the event makes it formal)
        if (flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[0], 0));
        MOKB_TRY(mokb_swiglu_bwd(a->gate_routed, a->up_routed, a->d_hidden_routed, a->d_gate_routed, a->d_up_routed, s.w_row, s.d_w_row,
                                 s.mb_rows + m, MB, I, lim, limv, stream));
        // d_x = d_gate * W_gate + d_up * W_up; the epilogue stores every row straight into slot t*K+k of its home rank's
        // d_x_routed buffer, and the route's router-weight gradient with it (the reverse dispatch)
        g = gemm_base(a->status);
        g.mode = 2; g.rows_static = hi; g.row_begin = lo; g.row_end = hi;
        g.num_rows = s.n_rows; g.group_of_block = s.group_of_block; g.G = E_l; g.N = H; g.K = I;
        g.A = d_gate_r; g.B = a->w_routed_gate; g.A2 = d_up_r; g.B2 = a->w_routed_up; g.lda = I; g.ldb = H;
        g.D = d_x_r; g.ldd = H;
        g.push_ptrs_host = a->d_x_routed_ptrs_host; g.push_ep_size = a->ep_size;
        g.push_rank = a->peer_rank; g.push_idx = a->peer_token_idx; g.push_index_limit = routes;
        g.push_values = d_w_row; g.push_value_ptrs_host = a->d_router_weight_ptrs_host;
        MOKB_TRY(mokb_grouped_gemm_bf16(&g, stream));
        const int32_t* offs = s.mb_offsets + static_cast<size_t>(m) * (E_l + 1);
        const int32_t* k_end = s.mb_k_end + static_cast<size_t>(m) * (E_l + 1);
        MOKB_TRY(wgrad(d_y_r, H, hidden_r, I, a->d_w_routed_down, E_l, hi, offs, m > 0, k_end));
        MOKB_TRY(wgrad(d_gate_r, I, x_routed, H, a->d_w_routed_gate, E_l, hi, offs, m > 0, k_end));
        MOKB_TRY(wgrad(d_up_r, I, x_routed, H, a->d_w_routed_up, E_l, hi, offs, m > 0, k_end));
    }
    return MOKB_OK;
}
