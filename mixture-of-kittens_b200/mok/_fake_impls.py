"""Meta ("fake") kernels of the `mok::` operators: output shapes and dtypes only, so
FakeTensor tracing and torch.compile(fullgraph=True) can capture the layer without
running device code (the role of mok/_fake_impls.py in the reference)."""
from __future__ import annotations

import torch

_registered = False


def _bf(x, *shape):
    return x.new_empty(shape, dtype=torch.bfloat16)


def register() -> None:
    global _registered
    if _registered:
        return
    _registered = True
    fake = torch.library.register_fake

    @fake("mok::all_gather_top_experts")
    def _(top_experts, buf, mc_ptr, rank, chunk_bytes, ptrs=None):
        return None

    @fake("mok::barrier_all")
    def _(barrier_buffer, ptrs, mc_ptr, target):
        return None

    @fake("mok::schedule")
    def _(topk_all, num_local_experts, schedule_capacity, rank):
        i32 = dict(dtype=torch.int32)
        return (topk_all.new_empty((schedule_capacity,), **i32), topk_all.new_empty((schedule_capacity,), **i32),
                topk_all.new_empty((1,), **i32), topk_all.new_empty((num_local_experts,), **i32))

    @fake("mok::mxfp8_quantize")
    def _(x_bf16, return_normal, return_transposed):
        lead = tuple(x_bf16.shape[:-2])
        E = lead[0] if lead else 1
        M, N = x_bf16.shape[-2:]
        q = s = qt = st = None
        if return_normal:
            q = x_bf16.new_empty((*lead, M, N), dtype=torch.float8_e4m3fn)
            s = x_bf16.new_empty((E * M // 128, N // 128, 32, 16), dtype=torch.uint8)
        if return_transposed:
            qt = x_bf16.new_empty((*lead, N, M), dtype=torch.float8_e4m3fn)
            st = x_bf16.new_empty((E * N // 128, M // 128, 32, 16), dtype=torch.uint8)
        return q, s, qt, st

    def fwd_shapes(x, w_shared_gate, macrobatch_size, with_down):
        T, H = x.shape
        I = w_shared_gate.shape[0]
        MB = macrobatch_size
        out = (_bf(x, MB, H), _bf(x, T, I), _bf(x, MB, I), _bf(x, T, I), _bf(x, MB, I), _bf(x, T, I), _bf(x, MB, I))
        if with_down:
            out += (_bf(x, T, H), _bf(x, MB, H))
        return out

    @fake("mok::dispatch_mlp_swiglu_combine_fwd_bf16")
    def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
          w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
          topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
        return fwd_shapes(x, w_shared_gate, macrobatch_size, True)

    @fake("mok::recompute_forward_context_bf16")
    def _(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank,
          schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
          minibatch_size):
        return fwd_shapes(x, w_shared_gate, macrobatch_size, False)

    @fake("mok::dispatch_mlp_swiglu_combine_bwd_bf16")
    def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
          router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate,
          w_shared_up, w_routed_up, w_shared_down, w_routed_down, x_routed, gate_shared, gate_routed, up_shared,
          up_routed, hidden_shared, hidden_routed, x, x_ptrs, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
          tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
        T, H = x.shape
        I = w_shared_gate.shape[0]
        E_l = w_routed_gate.shape[0]
        MB = macrobatch_size
        return (_bf(x, T, H), _bf(x, MB, H), _bf(x, T, I), _bf(x, MB, I), _bf(x, T, I), _bf(x, MB, I), _bf(x, T, I),
                _bf(x, MB, I), _bf(x, MB, H), _bf(x, I, H), _bf(x, E_l, I, H), _bf(x, I, H), _bf(x, E_l, I, H),
                _bf(x, H, I), _bf(x, E_l, H, I))

    @fake("mok::fwd_epilogue")
    def _(y_shared, combine_buffer, topk_weights):
        return torch.empty_like(y_shared)

    @fake("mok::bwd_epilogue")
    def _(d_x_shared, d_x_routed_buffer):
        return torch.empty_like(d_x_shared)
