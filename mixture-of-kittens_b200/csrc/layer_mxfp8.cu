#include "layer_common.cuh"

using namespace mokb;

// ============================================================================
// MXFP8: routed experts in block-scaled E4M3, shared expert in BF16
// (reference: csrc/megakernel/forward.cuh:296-428, backward.cuh:448-679).
//
// Dataflow (quantisation points as in the reference):
//   forward   dispatch x -> quantise x row-wise (GEMM operand) and token-wise (saved for wgrad)
//             gate, up = x_q * Wg_q^T, x_q * Wu_q^T, rounded to bf16 in the GEMM epilogue, which also applies SwiGLU
//             and quantises gate, up (saved) and hidden row-wise (GEMM operand) and token-wise (saved)
//             -> y = hidden_q * Wd_q^T -> combine
//   backward  pull d_y * w -> quantise both ways -> d_hidden = d_y_q * WdT_q^T
//             -> de-quantise saved gate/up, SwiGLU backward, router-gradient partials, quantise d_gate, d_up
//             both ways -> d_x = d_gate_q * WgT_q^T + d_up_q * WuT_q^T -> combine;
//             weight gradients contract the token-wise quantised tensors over each expert's rows.
//
// Macrobatches: every [MB, .] / [., MB] buffer holds the rows of one macrobatch at a time.  The forward walks
// the macrobatches last to first, so the buffers finally hold macrobatch 0 (the saved context); the backward
// starts with macrobatch 0 from the context and replays the later ones (dispatch x, quantise, gate|up,
// SwiGLU + quantise) into the same buffers, accumulating the weight gradients.  Kernels address rows by
// their schedule row number; a buffer's pointers are moved back by the macrobatch's first row.
//
// Overlap: macrobatch 0 of the forward is cut into row windows (minibatch_size rows): dispatch + quantise of
// window c+1 and the combine of window c-1 run on the side streams while the GEMMs of window c run on the
// caller's stream.  In the backward the d_y pull + quantisation comes in four windows behind the shared
// expert's BF16 GEMMs, the first routed GEMM follows it window by window, and the d_x push overlaps the
// weight gradients.
namespace mokb {
namespace {

mokb_gemm_fp8_args fp8_base(int32_t* status) {
    mokb_gemm_fp8_args g;
    memset(&g, 0, sizeof(g));
    g.G = 1;
    g.status = status;
    return g;
}

// Packed scale tensor [rows/128, cols/128, 32, 16] of a [rows, cols] matrix, moved back by `first` rows.
inline void* rebase_scales(const void* sc, int first, int cols) {
    return reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(sc) - static_cast<size_t>(first / 128) * (cols / 128) * 512);
}
// Token-wise ("transposed") E4M3 tensor [cols, MB], token r of the macrobatch at column r - first: moved back by `first` bytes;
// its scale tensor [cols/128, MB/128, 32, 16] by first/128 tiles.
inline void* rebase_t(const void* p, int first) {
    return reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(p) - static_cast<size_t>(first));
}
inline void* rebase_scales_t(const void* sc, int first) {
    return reinterpret_cast<void*>(reinterpret_cast<uintptr_t>(sc) - static_cast<size_t>(first / 128) * 512);
}

// The routed forward tensors of one macrobatch, addressed by schedule row.
struct FwdView {
    void *x_routed, *x_fp8, *x_sc, *x_fp8_t, *x_sc_t;
    void *gate_fp8, *gate_sc, *up_fp8, *up_sc;
    void *hidden_fp8, *hidden_sc, *hidden_fp8_t, *hidden_sc_t;
};

FwdView fwd_view(int lo, int H, int I, void* x_routed, void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t,
                 void* gate_fp8, void* gate_sc, void* up_fp8, void* up_sc, void* hidden_fp8, void* hidden_sc,
                 void* hidden_fp8_t, void* hidden_sc_t) {
    FwdView v;
    v.x_routed = rebase(x_routed, lo, 2ull * H);
    v.x_fp8 = rebase(x_fp8, lo, 1ull * H);
    v.x_sc = rebase_scales(x_sc, lo, H);
    v.x_fp8_t = rebase_t(x_fp8_t, lo);
    v.x_sc_t = rebase_scales_t(x_sc_t, lo);
    v.gate_fp8 = rebase(gate_fp8, lo, 1ull * I);
    v.gate_sc = rebase_scales(gate_sc, lo, I);
    v.up_fp8 = rebase(up_fp8, lo, 1ull * I);
    v.up_sc = rebase_scales(up_sc, lo, I);
    v.hidden_fp8 = rebase(hidden_fp8, lo, 1ull * I);
    v.hidden_sc = rebase_scales(hidden_sc, lo, I);
    v.hidden_fp8_t = rebase_t(hidden_fp8_t, lo);
    v.hidden_sc_t = rebase_scales_t(hidden_sc_t, lo);
    return v;
}

struct GateUpWeights {
    const void *gate, *gate_sc, *up, *up_sc;
};

// rows [r0, r1) of macrobatch rows [.., hi): gate|up GEMM whose epilogue applies SwiGLU and writes gate, up and hidden in MXFP8
int gate_up_swiglu(const FwdView& v, const GateUpWeights& w, const Scratch& s, int r0, int r1, int hi, int MB, int E_l, int H, int I,
                   int has_limit, float limit, int32_t* status, cudaStream_t stream) {
    mokb_gemm_fp8_args f = fp8_base(status);
    f.mode = 3; f.rows_static = hi; f.row_begin = r0; f.row_end = r1;
    f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
    f.A = v.x_fp8; f.A_sc = v.x_sc; f.B = w.gate; f.B_sc = w.gate_sc; f.B2 = w.up; f.B2_sc = w.up_sc;
    f.gate_q = v.gate_fp8; f.gate_sc = v.gate_sc; f.up_q = v.up_fp8; f.up_sc = v.up_sc;
    f.hid_q = v.hidden_fp8; f.hid_sc = v.hidden_sc; f.hid_qt = v.hidden_fp8_t; f.hid_sct = v.hidden_sc_t;
    f.t_rows = MB; f.has_swiglu_limit = has_limit; f.swiglu_limit = limit; f.ldd = I;
    return mokb_grouped_gemm_mxfp8(&f, stream);
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
    MOKB_REQUIRE(a->x_routed && a->x_fp8 && a->x_sc && a->hidden_fp8 && a->hidden_sc, "fwd_mxfp8: null work buffer");
    const bool with_down = !a->skip_down_combine;
    if (with_down)
        MOKB_REQUIRE(a->combine_ptrs_host && a->w_shared_down && a->w_routed_down && a->w_routed_down_sc && a->y_shared,
                     "fwd_mxfp8: null down/combine pointer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const int C = a->schedule_capacity;
    const int64_t routes = static_cast<int64_t>(T) * a->topk;      // every rank's routes are numbered [0, routes)
    const Scratch s = carve(a->scratch, C, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream;
    cudaStream_t s_q = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * kCommBlocksPerSm : 0;
    // recompute only rebuilds macrobatch 0 (the saved context); the forward walks all of them, last first
    const int n_macro = with_down ? macrobatches(C, MB) : 1;
    const GateUpWeights wgu{a->w_routed_gate, a->w_routed_gate_sc, a->w_routed_up, a->w_routed_up_sc};

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, a->peer_rank, E_l, C, MB, T, s, a->status, stream));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));
    bool shared_done = false;

    for (int mi = 0; mi < n_macro; ++mi) {
        const int m = n_macro - 1 - mi;
        const int lo = m * MB, hi = (lo + MB < C) ? lo + MB : C;
        // only macrobatch 0 (the one that is always populated) is cut into overlap windows, which are tied to the one
        // persistent GEMM launch by counters (layer.cu)
        const int chunk = m == 0 ? chunk_rows_for(MB, a->minibatch_size) : MB;
        const int nchunks = (hi - lo + chunk - 1) / chunk;
        const bool flags = overlap && m == 0;
        const FwdView v = fwd_view(lo, H, I, a->x_routed, a->x_fp8, a->x_sc, a->x_fp8_t, a->x_sc_t, a->gate_fp8,
                                   a->gate_sc, a->up_fp8, a->up_sc, a->hidden_fp8, a->hidden_sc, a->hidden_fp8_t, a->hidden_sc_t);
        void* y_r = (with_down && a->y_routed) ? rebase(a->y_routed, lo, 2ull * H) : nullptr;

        if (overlap) {     // everything enqueued so far (previous macrobatch included) precedes this one's side work
            MOKB_CUDA(cudaEventRecord(as->fork, stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        }
        // dispatch, window by window: the pull also quantises every row along its columns (what the GEMM reads) and
        // raises the window's counter; the token-wise form (for the weight gradients of the backward pass) follows
        // from the bf16 rows on a second, lower-priority side stream, window by window behind the pull, under the GEMM
        for (int c = 0; c < nchunks; ++c) {
            const int r0 = lo + c * chunk, r1 = r0 + chunk < hi ? r0 + chunk : hi;
            MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, r0, r1, a->topk, H,
                                        v.x_routed, nullptr, nullptr, comm_blocks, s_in, flags ? s.win_ready + c : nullptr,
                                        v.x_fp8, v.x_sc, routes, a->status));
            if (overlap) {
                MOKB_CUDA(cudaEventRecord(as->ev_in[c], s_in));
                MOKB_CUDA(cudaStreamWaitEvent(s_q, as->ev_in[c], 0));
            }
            MOKB_TRY(quantize_impl(v.x_routed, 1, MB, H, s.n_rows, r0, r1, nullptr, nullptr, v.x_fp8_t, v.x_sc_t, s_q, comm_blocks));
        }
        if (overlap) {
            MOKB_CUDA(cudaEventRecord(as->join1, s_in));
            MOKB_CUDA(cudaEventRecord(as->join2, s_q));
        }

        if (!shared_done) {
            // shared expert (BF16): gate/up + SwiGLU in one pass, then down (independent of the dispatch)
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

        // routed experts (MXFP8): gate|up + SwiGLU + quantisation and the down projection of every window in one launch;
        // the down epilogue stores every row into its home rank's combine buffer
        if (overlap && !flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
        mokb_gemm_fp8_args f = fp8_base(a->status);
        f.mode = 4; f.rows_static = hi; f.row_begin = lo; f.row_end = hi;
        f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
        f.A = v.x_fp8; f.A_sc = v.x_sc; f.B = wgu.gate; f.B_sc = wgu.gate_sc; f.B2 = wgu.up; f.B2_sc = wgu.up_sc;
        f.gate_q = v.gate_fp8; f.gate_sc = v.gate_sc; f.up_q = v.up_fp8; f.up_sc = v.up_sc;
        f.hid_q = v.hidden_fp8; f.hid_sc = v.hidden_sc; f.hid_qt = v.hidden_fp8_t; f.hid_sct = v.hidden_sc_t;
        f.t_rows = MB; f.has_swiglu_limit = a->has_swiglu_limit; f.swiglu_limit = a->swiglu_limit;
        f.window_rows = chunk;
        f.blk_done = s.blk_done + lo / 256;
        if (flags) { f.win_ready = s.win_ready; f.win_ready_target = comm_blocks; }
        f.ldd = H;
        if (with_down) {
            f.B3 = a->w_routed_down; f.B3_sc = a->w_routed_down_sc; f.N2 = H; f.D = y_r;
            f.push_ptrs_host = a->combine_ptrs_host; f.push_ep_size = a->ep_size;
            f.push_rank = a->peer_rank; f.push_idx = a->peer_token_idx; f.push_index_limit = routes;
        }
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        // the next macrobatch (or the caller) reuses the pulled rows: the side stream must be done with them
        if (flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
        // ... and with the token-wise copies, which are outputs of this call (and read the pulled rows)
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join2, 0));
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
    MOKB_REQUIRE(a->d_x_shared && a->d_gate_shared && a->d_gate_fp8 && a->d_gate_sc && a->d_up_shared && a->d_up_fp8 &&
                 a->d_up_sc && a->d_hidden_shared && a->d_hidden_routed && a->d_y_fp8 && a->d_y_sc && a->d_w_shared_gate &&
                 a->d_w_routed_gate && a->d_w_shared_up && a->d_w_routed_up && a->d_w_shared_down && a->d_w_routed_down, "bwd_mxfp8: null output");
    MOKB_REQUIRE(a->d_y_routed && a->d_y_fp8_t && a->d_y_sc_t && a->d_gate_fp8_t && a->d_gate_sc_t && a->d_up_fp8_t && a->d_up_sc_t && a->partials,
                 "bwd_mxfp8: null work buffer");
    const int T = a->num_local_tokens, H = a->hidden, I = a->intermediate, E_l = a->num_local_experts, MB = a->macrobatch_size;
    const int C = a->schedule_capacity;
    const int64_t routes = static_cast<int64_t>(T) * a->topk;      // every rank's routes are numbered [0, routes)
    const int n_macro = macrobatches(C, MB);
    if (n_macro > 1)
        MOKB_REQUIRE(a->w_routed_gate && a->w_routed_gate_sc && a->w_routed_up && a->w_routed_up_sc && a->x_routed && a->x_fp8 && a->x_sc &&
                     a->hidden_fp8 && a->hidden_sc,
                     "bwd_mxfp8: schedule_capacity > macrobatch_size needs the forward weights and the replay work buffers");
    const Scratch s = carve(a->scratch, C, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * kCommBlocksPerSm : 0;
    const int lim = a->has_swiglu_limit;
    const float limv = a->swiglu_limit;
    const GateUpWeights wgu{a->w_routed_gate, a->w_routed_gate_sc, a->w_routed_up, a->w_routed_up_sc};

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, a->peer_rank, E_l, C, MB, T, s, a->status, stream));
    const void* d_y_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->d_y_ptrs_host[a->ep_rank]));
    const void* x_local = reinterpret_cast<const void*>(static_cast<uintptr_t>(a->x_ptrs_host[a->ep_rank]));

    for (int m = 0; m < n_macro; ++m) {
        const int lo = m * MB, hi = (lo + MB < C) ? lo + MB : C;
        // the context (macrobatch 0: as saved; later ones: rebuilt below) and the work buffers, addressed by schedule row
        const FwdView v = fwd_view(lo, H, I, a->x_routed, a->x_fp8, a->x_sc, a->x_fp8_t, a->x_sc_t, a->gate_fp8,
                                   a->gate_sc, a->up_fp8, a->up_sc, a->hidden_fp8, a->hidden_sc, a->hidden_fp8_t, a->hidden_sc_t);
        void* d_y_r = rebase(a->d_y_routed, lo, 2ull * H);
        void* d_y_fp8 = rebase(a->d_y_fp8, lo, 1ull * H);
        void* d_y_sc = rebase_scales(a->d_y_sc, lo, H);
        void* d_y_fp8_t = rebase_t(a->d_y_fp8_t, lo);
        void* d_y_sc_t = rebase_scales_t(a->d_y_sc_t, lo);
        void* d_hidden_r = rebase(a->d_hidden_routed, lo, 2ull * I);
        void* d_gate_fp8 = rebase(a->d_gate_fp8, lo, 1ull * I);
        void* d_gate_sc = rebase_scales(a->d_gate_sc, lo, I);
        void* d_gate_fp8_t = rebase_t(a->d_gate_fp8_t, lo);
        void* d_gate_sc_t = rebase_scales_t(a->d_gate_sc_t, lo);
        void* d_up_fp8 = rebase(a->d_up_fp8, lo, 1ull * I);
        void* d_up_sc = rebase_scales(a->d_up_sc, lo, I);
        void* d_up_fp8_t = rebase_t(a->d_up_fp8_t, lo);
        void* d_up_sc_t = rebase_scales_t(a->d_up_sc_t, lo);
        void* d_x_r = a->d_x_routed ? rebase(a->d_x_routed, lo, 2ull * H) : nullptr;
        float* w_row = rebase(s.w_row, lo, 4);
        float* d_w_row = rebase(s.d_w_row, lo, 4);
        float* partials = rebase(static_cast<float*>(a->partials), lo, 4ull * (I / 128));

        if (overlap) {     // the previous macrobatch's weight gradients still read the buffers the dispatches below overwrite
            MOKB_CUDA(cudaEventRecord(as->fork, stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        }
        if (m > 0) {       // replay: pull x again and quantise it both ways
            MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, lo, hi, a->topk, H,
                                        v.x_routed, nullptr, nullptr, comm_blocks, s_in, nullptr, v.x_fp8, v.x_sc, routes, a->status));
            MOKB_TRY(quantize_impl(v.x_routed, 1, MB, H, s.n_rows, lo, hi, nullptr, nullptr, v.x_fp8_t, v.x_sc_t, s_in, comm_blocks));
        }
        if (overlap) MOKB_CUDA(cudaEventRecord(as->join1, s_in));     // the replayed x is in place
        // reverse combine: pull d_y rows scaled by the route's router weight and quantise them both ways, in a few windows
        // (macrobatch 0: the pull's blocks raise the window's counter for the one d_hidden launch below)
        const bool flags = overlap && m == 0;
        const int bchunk = bwd_chunk_rows(hi - lo, m == 0);
        const int nb = (hi - lo + bchunk - 1) / bchunk;
        for (int c = 0; c < nb; ++c) {
            const int r0 = lo + c * bchunk, r1 = r0 + bchunk < hi ? r0 + bchunk : hi;
            MOKB_TRY(dispatch_rows_impl(a->d_y_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, C, r0, r1, a->topk, H,
                                        d_y_r, a->router_weight_ptrs_host, w_row, comm_blocks, s_in, flags ? s.win_ready + c : nullptr,
                                        d_y_fp8, d_y_sc, routes, a->status));
        }
        if (overlap) MOKB_CUDA(cudaEventRecord(as->ev_in[0], s_in));
        for (int c = 0; c < nb; ++c) {       // the token-wise form of d_y, for the weight gradients at the end
            const int r0 = lo + c * bchunk, r1 = r0 + bchunk < hi ? r0 + bchunk : hi;
            MOKB_TRY(quantize_impl(d_y_r, 1, MB, H, s.n_rows, r0, r1, nullptr, nullptr, d_y_fp8_t, d_y_sc_t, s_in, comm_blocks));
        }
        if (overlap) MOKB_CUDA(cudaEventRecord(as->ev_in[1], s_in));

        if (m == 0) {
            // ---- shared expert (BF16; overlaps the dispatch above)
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
        }

        // ---- routed experts of this macrobatch (MXFP8)
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->join1, 0));
        if (m > 0)         // replay gate|up + SwiGLU + quantisation into the context buffers
            MOKB_TRY(gate_up_swiglu(v, wgu, s, lo, hi, hi, MB, E_l, H, I, lim, limv, a->status, stream));
        // d_hidden = d_y_q * WdT_q^T: one launch, window by window behind the pull
        if (overlap && !flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[0], 0));
        mokb_gemm_fp8_args f = fp8_base(a->status);
        f.mode = 0; f.rows_static = hi; f.row_begin = lo; f.row_end = hi;
        f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
        f.A = d_y_fp8; f.A_sc = d_y_sc; f.B = a->w_routed_down_t; f.B_sc = a->w_routed_down_t_sc; f.D = d_hidden_r; f.ldd = I;
        if (flags) { f.window_rows = bchunk; f.win_ready = s.win_ready; f.win_ready_target = comm_blocks; }
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        if (flags) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[0], 0));
        MOKB_TRY(swiglu_bwd_quant_impl(v.gate_fp8, v.gate_sc, v.up_fp8, v.up_sc, d_hidden_r, MB, I, s.n_rows, lo, hi, lim, limv, w_row,
                                       d_gate_fp8, d_gate_sc, d_gate_fp8_t, d_gate_sc_t, d_up_fp8, d_up_sc, d_up_fp8_t, d_up_sc_t,
                                       partials, d_w_row, stream));
        f = fp8_base(a->status);
        f.mode = 0; f.rows_static = hi; f.row_begin = lo; f.row_end = hi;
        f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = H; f.K = I;
        f.A = d_gate_fp8; f.A_sc = d_gate_sc; f.B = a->w_routed_gate_t; f.B_sc = a->w_routed_gate_t_sc;
        f.A2 = d_up_fp8; f.A2_sc = d_up_sc; f.B2 = a->w_routed_up_t; f.B2_sc = a->w_routed_up_t_sc; f.D = d_x_r; f.ldd = H;
        // reverse dispatch: the epilogue stores every d_x row and its router-weight gradient into the home rank's buffers
        f.push_ptrs_host = a->d_x_routed_ptrs_host; f.push_ep_size = a->ep_size;
        f.push_rank = a->peer_rank; f.push_idx = a->peer_token_idx; f.push_index_limit = routes;
        f.push_values = d_w_row; f.push_value_ptrs_host = a->d_router_weight_ptrs_host;
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        const int32_t* offs = s.mb_offsets + static_cast<size_t>(m) * (E_l + 1);
        auto wgrad_fp8 = [&](const void* A, const void* A_sc, int M, const void* B, const void* B_sc, int N, void* D) -> int {
            mokb_gemm_fp8_args w = fp8_base(a->status);
            w.mode = 2; w.rows_static = MB; w.t_first = lo; w.G = E_l; w.M = M; w.N = N; w.group_offsets = offs; w.accumulate = m > 0;
            w.A = A; w.A_sc = A_sc; w.B = B; w.B_sc = B_sc; w.D = D; w.ldd = N;
            return mokb_grouped_gemm_mxfp8(&w, stream);
        };
        // the token-wise tensors are passed as they lie in memory ([., MB], first token column = lo)
        MOKB_TRY(wgrad_fp8(a->d_gate_fp8_t, a->d_gate_sc_t, I, a->x_fp8_t, a->x_sc_t, H, a->d_w_routed_gate));
        MOKB_TRY(wgrad_fp8(a->d_up_fp8_t, a->d_up_sc_t, I, a->x_fp8_t, a->x_sc_t, H, a->d_w_routed_up));
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[1], 0));      // the token-wise d_y is complete
        MOKB_TRY(wgrad_fp8(a->d_y_fp8_t, a->d_y_sc_t, H, a->hidden_fp8_t, a->hidden_sc_t, I, a->d_w_routed_down));
    }
    return MOKB_OK;
}
