"""The MXFP8 operators of `mok.ops` (reference: mok/ops.py:200-374, 523-665, 785-1076): same names,
argument order, mutation schemas and exceptions.  `mok.ops` re-exports them."""
import torch

from . import _C_mxfp8
from . import ops as _ops

F8 = torch.float8_e4m3fn


def _sc_shape(rows: int, cols: int) -> tuple[int, int, int, int]:
    return (rows // 128, cols // 128, 32, 16)


def _validate_common(x, x_ptrs, w_shared_gate, w_routed_gate, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
                     tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
    T, H = _ops._check_activation("x", x)
    if w_shared_gate.ndim != 2:
        raise ValueError("w_shared_gate must have shape (intermediate_size, hidden_size)")
    I, E_l = _ops._check_weights(w_shared_gate, w_routed_gate, H)
    _ops._check_knobs(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _ops._check_ptrs("x_ptrs", x_ptrs)
    _ops._check_schedule(schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, E_l)
    return T, H, I, E_l, ep_size


def _check_table(device, table):
    for name, t, shape, dtype in table:
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name} must have shape {tuple(shape)}")
        if dtype is not None and t.dtype != dtype:
            raise TypeError(f"{name} must have dtype {dtype}")
    for name, t, _, _ in table:
        if t.device != device:
            raise ValueError(f"{name} must be on {device}")


@_ops._op("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_mxfp8(
    x: torch.Tensor,
    x_ptrs: list[int],
    combine_buffer: torch.Tensor,
    combine_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
    w_routed_down_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fused MXFP8 forward.  Returns x_fp8_t_routed [H, MB], x_sc_t_routed, gate_shared [T, I], gate_fp8_routed
    [MB, I], gate_sc_routed, up_shared, up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed [I, MB],
    hidden_sc_t_routed, y_shared [T, H], y_routed [MB, H]; writes every peer's combine_buffer."""
    T, H, I, E_l, ep_size = _validate_common(x, x_ptrs, w_shared_gate, w_routed_gate, schedule_peer_rank,
                                             schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                                             num_comm_sms, macrobatch_size, minibatch_size)
    _ops._check_ptrs("combine_buffer_ptrs", combine_buffer_ptrs, ep_size)
    _check_table(x.device, [
        ("combine_buffer", combine_buffer, (T * topk, H), None),
        ("w_shared_gate", w_shared_gate, (I, H), None),
        ("w_routed_gate", w_routed_gate, (E_l, I, H), F8), ("w_routed_gate_sc", w_routed_gate_sc, _sc_shape(E_l * I, H), torch.uint8),
        ("w_shared_up", w_shared_up, (I, H), None),
        ("w_routed_up", w_routed_up, (E_l, I, H), F8), ("w_routed_up_sc", w_routed_up_sc, _sc_shape(E_l * I, H), torch.uint8),
        ("w_shared_down", w_shared_down, (H, I), None),
        ("w_routed_down", w_routed_down, (E_l, H, I), F8), ("w_routed_down_sc", w_routed_down_sc, _sc_shape(E_l * H, I), torch.uint8),
    ])
    return _C_mxfp8.dispatch_mlp_swiglu_combine_fwd_mxfp8(
        x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up,
        w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc, schedule_peer_rank,
        schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
        minibatch_size)


@_ops._op("mok::recompute_forward_context_mxfp8", mutates_args=())
def recompute_forward_context_mxfp8(
    x: torch.Tensor,
    x_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Forward without the down projection and combine: the first 11 outputs of the MXFP8 forward, bit-identical."""
    T, H, I, E_l, ep_size = _validate_common(x, x_ptrs, w_shared_gate, w_routed_gate, schedule_peer_rank,
                                             schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                                             num_comm_sms, macrobatch_size, minibatch_size)
    _check_table(x.device, [
        ("w_shared_gate", w_shared_gate, (I, H), None),
        ("w_routed_gate", w_routed_gate, (E_l, I, H), F8), ("w_routed_gate_sc", w_routed_gate_sc, _sc_shape(E_l * I, H), torch.uint8),
        ("w_shared_up", w_shared_up, (I, H), None),
        ("w_routed_up", w_routed_up, (E_l, I, H), F8), ("w_routed_up_sc", w_routed_up_sc, _sc_shape(E_l * I, H), torch.uint8),
    ])
    return _C_mxfp8.recompute_forward_context_mxfp8(
        x, x_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up, w_routed_up, w_routed_up_sc,
        schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
        macrobatch_size, minibatch_size)


@_ops._op(
    "mok::dispatch_mlp_swiglu_combine_bwd_mxfp8",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_fp8_t_routed", "x_sc_t_routed", "gate_fp8_routed",
                  "gate_sc_routed", "up_fp8_routed", "up_sc_routed", "hidden_fp8_t_routed", "hidden_sc_t_routed"),
)
def dispatch_mlp_swiglu_combine_bwd_mxfp8(
    d_y_buffer: torch.Tensor,
    d_y_buffer_ptrs: list[int],
    d_x_routed_buffer: torch.Tensor,
    d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: torch.Tensor,
    router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: torch.Tensor,
    d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate_T: torch.Tensor,
    w_routed_gate_T_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up_T: torch.Tensor,
    w_routed_up_T_sc: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down_T: torch.Tensor,
    w_routed_down_T_sc: torch.Tensor,
    x_fp8_t_routed: torch.Tensor,
    x_sc_t_routed: torch.Tensor,
    gate_shared: torch.Tensor,
    gate_fp8_routed: torch.Tensor,
    gate_sc_routed: torch.Tensor,
    up_shared: torch.Tensor,
    up_fp8_routed: torch.Tensor,
    up_sc_routed: torch.Tensor,
    hidden_shared: torch.Tensor,
    hidden_fp8_t_routed: torch.Tensor,
    hidden_sc_t_routed: torch.Tensor,
    x: torch.Tensor,
    x_ptrs: list[int],
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fused MXFP8 backward.  Returns d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8_routed, d_gate_sc_routed,
    d_up_shared, d_up_fp8_routed, d_up_sc_routed, d_hidden_shared, d_hidden_routed, d_y_fp8_routed, d_y_sc_routed,
    d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down."""
    T, H, I, E_l, ep_size = _validate_common(x, x_ptrs, w_shared_gate, w_routed_gate, schedule_peer_rank,
                                             schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                                             num_comm_sms, macrobatch_size, minibatch_size)
    for name, ptrs in (("d_y_buffer_ptrs", d_y_buffer_ptrs), ("d_x_routed_buffer_ptrs", d_x_routed_buffer_ptrs),
                       ("router_weight_buffer_ptrs", router_weight_buffer_ptrs),
                       ("d_router_weight_buffer_ptrs", d_router_weight_buffer_ptrs)):
        _ops._check_ptrs(name, ptrs, ep_size)
    MB = macrobatch_size
    u8 = torch.uint8
    _check_table(x.device, [
        ("d_y_buffer", d_y_buffer, (T, H), None), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H), None),
        ("router_weight_buffer", router_weight_buffer, (T, topk), None),
        ("d_router_weight_buffer", d_router_weight_buffer, (T, topk), None),
        ("w_shared_gate", w_shared_gate, (I, H), None), ("w_shared_up", w_shared_up, (I, H), None),
        ("w_shared_down", w_shared_down, (H, I), None),
        ("w_routed_gate_T", w_routed_gate_T, (E_l, H, I), F8), ("w_routed_gate_T_sc", w_routed_gate_T_sc, _sc_shape(E_l * H, I), u8),
        ("w_routed_up_T", w_routed_up_T, (E_l, H, I), F8), ("w_routed_up_T_sc", w_routed_up_T_sc, _sc_shape(E_l * H, I), u8),
        ("w_routed_down_T", w_routed_down_T, (E_l, I, H), F8), ("w_routed_down_T_sc", w_routed_down_T_sc, _sc_shape(E_l * I, H), u8),
        ("x_fp8_t_routed", x_fp8_t_routed, (H, MB), F8), ("x_sc_t_routed", x_sc_t_routed, _sc_shape(H, MB), u8),
        ("gate_shared", gate_shared, (T, I), None), ("up_shared", up_shared, (T, I), None),
        ("hidden_shared", hidden_shared, (T, I), None),
        ("gate_fp8_routed", gate_fp8_routed, (MB, I), F8), ("gate_sc_routed", gate_sc_routed, _sc_shape(MB, I), u8),
        ("up_fp8_routed", up_fp8_routed, (MB, I), F8), ("up_sc_routed", up_sc_routed, _sc_shape(MB, I), u8),
        ("hidden_fp8_t_routed", hidden_fp8_t_routed, (I, MB), F8), ("hidden_sc_t_routed", hidden_sc_t_routed, _sc_shape(I, MB), u8),
        ("w_routed_gate", w_routed_gate, (E_l, I, H), F8), ("w_routed_gate_sc", w_routed_gate_sc, _sc_shape(E_l * I, H), u8),
        ("w_routed_up", w_routed_up, (E_l, I, H), F8), ("w_routed_up_sc", w_routed_up_sc, _sc_shape(E_l * I, H), u8),
    ])
    return _C_mxfp8.dispatch_mlp_swiglu_combine_bwd_mxfp8(
        d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
        router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs,
        w_shared_gate, w_routed_gate_T, w_routed_gate_T_sc, w_shared_up, w_routed_up_T, w_routed_up_T_sc,
        w_shared_down, w_routed_down_T, w_routed_down_T_sc,
        x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared, up_fp8_routed,
        up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed, x, x_ptrs,
        w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc,
        schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
        macrobatch_size, minibatch_size)


def _register_fakes() -> None:
    fake = torch.library.register_fake

    def q(x, rows, cols):
        return (x.new_empty((rows, cols), dtype=F8), x.new_empty(_sc_shape(rows, cols), dtype=torch.uint8))

    def bf(x, *shape):
        return x.new_empty(shape, dtype=torch.bfloat16)

    def fwd(x, w_shared_gate, MB, with_down):
        T, H = x.shape
        I = w_shared_gate.shape[0]
        out = (*q(x, H, MB), bf(x, T, I), *q(x, MB, I), bf(x, T, I), *q(x, MB, I), bf(x, T, I), *q(x, I, MB))
        return out + ((bf(x, T, H), bf(x, MB, H)) if with_down else ())

    @fake("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8")
    def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up,
          w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc, schedule_peer_rank,
          schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
          minibatch_size):
        return fwd(x, w_shared_gate, macrobatch_size, True)

    @fake("mok::recompute_forward_context_mxfp8")
    def _(x, x_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up, w_routed_up, w_routed_up_sc,
          schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
          macrobatch_size, minibatch_size):
        return fwd(x, w_shared_gate, macrobatch_size, False)

    @fake("mok::dispatch_mlp_swiglu_combine_bwd_mxfp8")
    def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
          router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate,
          w_routed_gate_T, w_routed_gate_T_sc, w_shared_up, w_routed_up_T, w_routed_up_T_sc, w_shared_down,
          w_routed_down_T, w_routed_down_T_sc, x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed,
          gate_sc_routed, up_shared, up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed,
          hidden_sc_t_routed, x, x_ptrs, w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc,
          schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
          num_comm_sms, macrobatch_size, minibatch_size):
        T, H = x.shape
        I = w_shared_gate.shape[0]
        E_l = w_routed_gate.shape[0]
        MB = macrobatch_size
        return (bf(x, T, H), bf(x, MB, H), bf(x, T, I), *q(x, MB, I), bf(x, T, I), *q(x, MB, I), bf(x, T, I),
                bf(x, MB, I), *q(x, MB, H), bf(x, I, H), bf(x, E_l, I, H), bf(x, I, H), bf(x, E_l, I, H), bf(x, H, I),
                bf(x, E_l, H, I))


_register_fakes()
