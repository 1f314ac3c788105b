#include "layer_common.cuh"

using namespace mokb;

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
// The forward is cut into row windows (minibatch_size rows each): dispatch + quantise of window c+1 and the
// combine of window c-1 run on the side streams while the GEMMs of window c run on the caller's stream.
// In the backward, dispatch / combine overlap the shared expert's BF16 GEMMs and the weight gradients.
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
    const Scratch s = carve(a->scratch, a->schedule_capacity, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream, s_out = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;
    // overlap windows: rows [r0, r1) flow dispatch+quantise (side stream 1) -> GEMMs (caller's stream) -> combine (side stream 2)
    const int chunk = chunk_rows_for(MB, a->minibatch_size);
    const int nchunks = (MB + chunk - 1) / chunk;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, true, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
        if (with_down) MOKB_CUDA(cudaStreamWaitEvent(s_out, as->fork, 0));
    }
    // dispatch + quantise (row-wise for the GEMM, token-wise for the weight gradients), window by window
    for (int c = 0; c < nchunks; ++c) {
        const int r0 = c * chunk, r1 = r0 + chunk < MB ? r0 + chunk : MB;
        MOKB_TRY(dispatch_rows_impl(a->x_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, r0, r1, a->topk, H,
                                    a->x_routed, nullptr, nullptr, comm_blocks, s_in));
        MOKB_TRY(quantize_impl(a->x_routed, 1, MB, H, s.n_rows, r0, r1, a->x_fp8, a->x_sc, a->x_fp8_t, a->x_sc_t, s_in));
        if (overlap) MOKB_CUDA(cudaEventRecord(as->ev_in[c], s_in));
    }
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

    // routed experts (MXFP8), window by window behind the dispatch
    for (int c = 0; c < nchunks; ++c) {
        const int r0 = c * chunk, r1 = r0 + chunk < MB ? r0 + chunk : MB;
        if (overlap) MOKB_CUDA(cudaStreamWaitEvent(stream, as->ev_in[c], 0));
        mokb_gemm_fp8_args f = fp8_base(a->status);
        f.mode = 1; f.rows_static = MB; f.row_begin = r0; f.row_end = r1;
        f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = I; f.K = H;
        f.A = a->x_fp8; f.A_sc = a->x_sc; f.B = a->w_routed_gate; f.B_sc = a->w_routed_gate_sc; f.B2 = a->w_routed_up; f.B2_sc = a->w_routed_up_sc;
        f.D = a->gate_bf16; f.D2 = a->up_bf16; f.ldd = I;
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        MOKB_TRY(swiglu_fwd_quant_impl(a->gate_bf16, a->up_bf16, MB, I, s.n_rows, r0, r1, a->has_swiglu_limit, a->swiglu_limit, a->gate_fp8,
                                       a->gate_sc, a->up_fp8, a->up_sc, a->hidden_fp8, a->hidden_sc, a->hidden_fp8_t, a->hidden_sc_t, stream));
        if (!with_down) continue;
        f = fp8_base(a->status);
        f.mode = 0; f.rows_static = MB; f.row_begin = r0; f.row_end = r1;
        f.num_rows = s.n_rows; f.group_of_block = s.group_of_block; f.G = E_l; f.N = H; f.K = I;
        f.A = a->hidden_fp8; f.A_sc = a->hidden_sc; f.B = a->w_routed_down; f.B_sc = a->w_routed_down_sc; f.D = a->y_routed; f.ldd = H;
        MOKB_TRY(mokb_grouped_gemm_mxfp8(&f, stream));
        if (overlap) {
            MOKB_CUDA(cudaEventRecord(as->ev_out[c], stream));
            MOKB_CUDA(cudaStreamWaitEvent(s_out, as->ev_out[c], 0));
        }
        MOKB_TRY(combine_rows_impl(a->y_routed, a->combine_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, r0, r1, H,
                                   nullptr, nullptr, comm_blocks, s_out));
    }
    if (overlap && with_down) {
        MOKB_CUDA(cudaEventRecord(as->join2, s_out));
        MOKB_CUDA(cudaStreamWaitEvent(stream, as->join2, 0));
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
    const Scratch s = carve(a->scratch, a->schedule_capacity, E_l, MB);
    const bool overlap = overlap_enabled();
    Async* as = nullptr;
    if (overlap) MOKB_TRY(get_async(&as));
    cudaStream_t s_in = overlap ? as->s1 : stream, s_out = overlap ? as->s2 : stream;
    const int comm_blocks = overlap ? a->num_comm_sms * 8 : 0;
    const int lim = a->has_swiglu_limit;
    const float limv = a->swiglu_limit;

    MOKB_TRY(run_prologue(a->tokens_per_expert, a->num_tokens, E_l, a->schedule_capacity, MB, T, true, s, a->status, stream));
    if (overlap) {
        MOKB_CUDA(cudaEventRecord(as->fork, stream));
        MOKB_CUDA(cudaStreamWaitEvent(s_in, as->fork, 0));
    }
    MOKB_TRY(dispatch_rows_impl(a->d_y_ptrs_host, a->ep_size, a->peer_rank, a->peer_token_idx, s.n_rows, MB, 0, MB, a->topk, H,
                                a->d_y_routed, a->router_weight_ptrs_host, s.w_row, comm_blocks, s_in));
    MOKB_TRY(quantize_impl(a->d_y_routed, 1, MB, H, s.n_rows, 0, MB, a->d_y_fp8, a->d_y_sc, a->d_y_fp8_t, a->d_y_sc_t, s_in));
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
    MOKB_TRY(swiglu_bwd_quant_impl(a->gate_fp8, a->gate_sc, a->up_fp8, a->up_sc, a->d_hidden_routed, MB, I, s.n_rows, 0, MB, lim, limv, s.w_row,
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
