"""`mok.ops`: the operator layer of the reference (mok/ops.py there), same operator
names under the `mok::` namespace, same argument order and meaning, same
mutation schemas, same error behaviour (ValueError / TypeError raised before any
device work) -- over the B200-native kernels of libmok_b200.so.

Differences a caller can see:
  * EP sizes: any size in [1, 64] (the reference: 1, 4, 8, 16, 32, 64), and
    intermediate_size may be any multiple of 128 (the reference: 256);
  * `all_gather_top_experts` and `barrier_all` take one optional trailing argument
    (the peers' unicast addresses / this rank's index) because they use plain peer
    stores instead of an NVLS multicast object;
  * a schedule that does not fit sets a device status word (mok._C.check_status)
    instead of trapping the GPU.
"""
import inspect

import torch

from . import _C
from . import _fake_impls

MAX_EP = 64

# operator -> (its Python body, positions of the arguments it mutates): what `call` needs to run it without the dispatcher
_EAGER: dict = {}


def _op(name: str, *, mutates_args=(), **kw):
    """`torch.library.custom_op` that also remembers the operator's body for `call`."""
    def deco(fn):
        op = torch.library.custom_op(name, mutates_args=mutates_args, **kw)(fn)
        params = list(inspect.signature(fn).parameters)
        _EAGER[op] = (fn, tuple(params.index(m) for m in mutates_args))
        return op
    return deco


# the three probes `_plain_eager` needs; a torch without them never takes the direct path
_dispatch_depth = getattr(torch._C, "_len_torch_dispatch_stack", None)
_function_depth = getattr(torch._C, "_len_torch_function_stack", None)
_functorch_top = getattr(getattr(torch._C, "_functorch", None), "peek_interpreter_stack", None)
_CAN_PROBE = None not in (_dispatch_depth, _function_depth, _functorch_top)


def _plain_eager(args) -> bool:
    if not _CAN_PROBE or torch.compiler.is_compiling() or _dispatch_depth() or _function_depth():
        return False
    if _functorch_top() is not None:
        return False
    for a in args:
        if isinstance(a, torch.Tensor) and (type(a) is not torch.Tensor or a.requires_grad):
            return False
    return True


def call(op, *args):
    """How `mok.functional` invokes an operator.  Under `torch.compile`, a dispatch or function mode (FakeTensorMode,
    make_fx, ...), a functorch transform, or with tensor subclasses / tensors that require grad, this is `op(*args)`.
    In plain eager mode the operator's body runs directly and the version counters of the arguments it mutates are
    bumped as the dispatcher would do: one dispatcher round trip costs about as much host time as launching ten small
    kernels, and a layer step makes eleven of them."""
    if not _plain_eager(args):
        return op(*args)
    fn, mutated = _EAGER[op]
    out = fn(*args)
    for i in mutated:
        if i < len(args) and args[i] is not None:
            torch.autograd.graph.increment_version(args[i])
    return out


def _is_pos_int(v) -> bool:
    return type(v) is int and v > 0


def _check_ptrs(name: str, ptrs, ep_size: int | None = None) -> int:
    if not isinstance(ptrs, list) or any(type(p) is not int or p <= 0 for p in ptrs):
        raise TypeError(f"{name} must be a list of positive integers")
    if not 1 <= len(ptrs) <= MAX_EP:
        raise ValueError(f"{name} length must be in [1, {MAX_EP}]")
    if ep_size is not None and len(ptrs) != ep_size:
        raise ValueError(f"{name} length must match x_ptrs")
    return len(ptrs)


def _check_knobs(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size) -> None:
    if type(topk) is not int or not 0 < topk <= 255:
        raise ValueError("topk must be an integer in [1, 255]")
    if swiglu_limit is not None and (type(swiglu_limit) not in (int, float) or swiglu_limit < 0):
        raise ValueError("swiglu_limit must be None or a non-negative number")
    if not _is_pos_int(num_comm_sms) or num_comm_sms % 2 != 0:
        raise ValueError("num_comm_sms must be a positive even integer")
    if not _is_pos_int(minibatch_size) or minibatch_size % 256 != 0:
        raise ValueError("minibatch_size must be positive and divisible by 256")
    if not _is_pos_int(macrobatch_size) or macrobatch_size % minibatch_size != 0:
        raise ValueError("macrobatch_size must be a positive multiple of minibatch_size")


def _check_activation(name: str, x: torch.Tensor) -> tuple[int, int]:
    if x.ndim != 2:
        raise ValueError(f"{name} must have shape (num_local_tokens, hidden_size)")
    T, H = x.shape
    if T < 512 or T % 256 != 0:
        raise ValueError("num_local_tokens must be at least 512 and divisible by 256")
    if H <= 0 or H % 256 != 0:
        raise ValueError("hidden_size must be positive and divisible by 256")
    return T, H


def _check_weights(w_shared_gate, w_routed_gate, hidden_size) -> tuple[int, int]:
    if w_shared_gate.ndim != 2 or w_shared_gate.shape[1] != hidden_size:
        raise ValueError("w_shared_gate must have shape (intermediate_size, hidden_size)")
    I = w_shared_gate.shape[0]
    if I <= 0 or I % 128 != 0:
        raise ValueError("intermediate_size must be positive and divisible by 128")
    if w_routed_gate.ndim != 3 or w_routed_gate.shape[0] <= 0:
        raise ValueError("w_routed_gate must have shape (num_local_experts, intermediate_size, hidden_size)")
    return I, w_routed_gate.shape[0]


def _check_schedule(peer_rank, peer_token_idx, num_tokens, tokens_per_expert, E_l) -> int:
    if peer_rank.ndim != 1 or peer_rank.numel() == 0:
        raise ValueError("schedule_peer_rank must be a nonempty 1D tensor")
    C = peer_rank.numel()
    if C % 256 != 0:
        raise ValueError("schedule_capacity must be divisible by 256")
    for name, t, shape in (("schedule_peer_token_idx", peer_token_idx, (C,)), ("num_tokens", num_tokens, (1,)),
                           ("tokens_per_expert", tokens_per_expert, (E_l,))):
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} must have shape {shape}")
    return C


def _check_shapes_devices(device, table) -> None:
    for name, t, shape in table:
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name} must have shape {tuple(shape)}")
    for name, t, _ in table:
        if t.device != device:
            raise ValueError(f"{name} must be on {device}")


@_op("mok::all_gather_top_experts", mutates_args=("all_gather_top_experts_buffer",))
def all_gather_top_experts(
    top_experts: torch.Tensor,
    all_gather_top_experts_buffer: torch.Tensor,
    all_gather_top_experts_buffer_multicast_ptr: int,
    rank: int,
    chunk_bytes: int,
    all_gather_top_experts_buffer_ptrs: list[int] | None = None,
) -> None:
    """All-gathers int32 [num_local_tokens, topk] routes into every rank's
    [ep_size, num_local_tokens, topk] buffer (reference: mok/ops.py:6-61)."""
    if not top_experts.is_cuda or top_experts.dtype != torch.int32 or not top_experts.is_contiguous() or top_experts.ndim != 2:
        raise ValueError("top_experts must be contiguous CUDA int32 [num_local_tokens, topk]")
    buf = all_gather_top_experts_buffer
    if not buf.is_cuda:
        raise ValueError("all_gather_top_experts_buffer must be a CUDA tensor")
    if buf.dtype != torch.int32:
        raise TypeError("all_gather_top_experts_buffer must have dtype torch.int32")
    if not buf.is_contiguous():
        raise ValueError("all_gather_top_experts_buffer must be contiguous")
    if buf.ndim != 3:
        raise ValueError("all_gather_top_experts_buffer must have shape (ep_size, num_local_tokens, topk)")
    if any(s <= 0 for s in top_experts.shape) or any(s <= 0 for s in buf.shape):
        raise ValueError("top_experts and all_gather_top_experts_buffer dimensions must be positive")
    ep_size = buf.shape[0]
    if not 1 <= ep_size <= MAX_EP:
        raise ValueError(f"all_gather_top_experts_buffer ep_size must be in [1, {MAX_EP}]")
    if buf.device != top_experts.device or tuple(buf.shape[1:]) != tuple(top_experts.shape):
        raise ValueError("all_gather_top_experts_buffer must match top_experts shape and device")
    if type(all_gather_top_experts_buffer_multicast_ptr) is not int or all_gather_top_experts_buffer_multicast_ptr < 0:
        raise TypeError("all_gather_top_experts_buffer_multicast_ptr must be a non-negative integer")
    if type(rank) is not int or not 0 <= rank < ep_size:
        raise ValueError("rank must be an integer in [0, ep_size)")
    if not _is_pos_int(chunk_bytes):
        raise ValueError("chunk_bytes must be a positive integer")
    if chunk_bytes % 16 != 0:
        raise ValueError("chunk_bytes must be divisible by 16")
    if (top_experts.numel() * 4) % chunk_bytes != 0:
        raise ValueError("chunk_bytes must divide one rank's route-buffer bytes")
    if ep_size == 1:
        buf[0].copy_(top_experts)
        return
    if all_gather_top_experts_buffer_ptrs is None:
        raise ValueError("all_gather_top_experts_buffer_ptrs is required when ep_size > 1")
    _check_ptrs("all_gather_top_experts_buffer_ptrs", all_gather_top_experts_buffer_ptrs)
    if len(all_gather_top_experts_buffer_ptrs) != ep_size:
        raise ValueError("all_gather_top_experts_buffer_ptrs length must equal ep_size")
    _C.all_gather_top_experts(top_experts, buf, all_gather_top_experts_buffer_multicast_ptr, rank, chunk_bytes,
                              all_gather_top_experts_buffer_ptrs)


@_op("mok::barrier_all", mutates_args=("barrier_buffer", "target"))
def barrier_all(
    barrier_buffer: torch.Tensor,
    barrier_buffer_ptrs: list[int],
    barrier_buffer_multicast_ptr: int,
    target: torch.Tensor,
) -> None:
    """Device-side barrier over all EP ranks (reference: mok/ops.py:64-106)."""
    if not barrier_buffer.is_cuda:
        raise ValueError("barrier_buffer must be a CUDA tensor")
    if barrier_buffer.dtype != torch.int32:
        raise TypeError("barrier_buffer must have dtype torch.int32")
    if not barrier_buffer.is_contiguous():
        raise ValueError("barrier_buffer must be contiguous")
    if tuple(barrier_buffer.shape) != (1,):
        raise ValueError("barrier_buffer must have shape (1,)")
    ep_size = _check_ptrs("barrier_buffer_ptrs", barrier_buffer_ptrs)
    if type(barrier_buffer_multicast_ptr) is not int or barrier_buffer_multicast_ptr < 0:
        raise TypeError("barrier_buffer_multicast_ptr must be a non-negative integer")
    if (not target.is_cuda or target.device != barrier_buffer.device or target.dtype != torch.int32
            or not target.is_contiguous() or tuple(target.shape) != (1,)):
        raise ValueError("target must be contiguous int32 [1] on the barrier CUDA device")
    if ep_size == 1:
        return
    if barrier_buffer.data_ptr() not in barrier_buffer_ptrs:
        raise ValueError("barrier_buffer's own address must appear in barrier_buffer_ptrs")
    _C.barrier_all(barrier_buffer, barrier_buffer_ptrs, barrier_buffer_multicast_ptr, target)


@_op("mok::schedule", mutates_args=())
def schedule(
    topk_all: torch.Tensor,
    num_local_experts: int,
    schedule_capacity: int,
    rank: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """int32 [ep_size, num_local_tokens, topk] -> (schedule_peer_rank [C], schedule_peer_token_idx [C],
    num_tokens [1], tokens_per_expert [num_local_experts]) (reference: mok/ops.py:109-156)."""
    if topk_all.ndim != 3:
        raise ValueError("topk_all must have shape (ep_size, num_local_tokens, topk)")
    if not topk_all.is_cuda or topk_all.dtype != torch.int32 or not topk_all.is_contiguous():
        raise ValueError("topk_all must be a contiguous CUDA int32 tensor")
    ep_size, T, K = topk_all.shape
    if not 1 <= ep_size <= MAX_EP:
        raise ValueError(f"topk_all ep_size must be in [1, {MAX_EP}]")
    if T < 512 or T % 256 != 0:
        raise ValueError("topk_all num_local_tokens must be at least 512 and divisible by 256")
    if not 0 < K <= 255:
        raise ValueError("topk_all topk must be in [1, 255]")
    if not _is_pos_int(num_local_experts):
        raise ValueError("num_local_experts must be a positive integer")
    if not _is_pos_int(schedule_capacity) or schedule_capacity % 256 != 0:
        raise ValueError("schedule_capacity must be positive and divisible by 256")
    if schedule_capacity < T * K:
        raise ValueError("schedule_capacity must hold at least one rank's routed tokens")
    if type(rank) is not int or not 0 <= rank < ep_size:
        raise ValueError("rank must be an integer in [0, ep_size)")
    return _C.schedule(topk_all, num_local_experts, schedule_capacity, rank)


@_op(
    "mok::mxfp8_quantize", mutates_args=(),
    schema="(Tensor x_bf16, bool return_normal, bool return_transposed) -> (Tensor?, Tensor?, Tensor?, Tensor?)",
)
def mxfp8_quantize(x_bf16, return_normal, return_transposed):
    """bf16 [M, N] or [E, M, N] -> (x_fp8, x_sc, x_fp8_t, x_sc_t) (reference: mok/ops.py:159-197)."""
    if x_bf16.ndim not in (2, 3):
        raise ValueError("x_bf16 must have shape (M, N) or (E, M, N)")
    if any(s <= 0 for s in x_bf16.shape):
        raise ValueError("x_bf16 dimensions must be positive")
    if x_bf16.shape[-2] % 128 != 0 or x_bf16.shape[-1] % 128 != 0:
        raise ValueError("x_bf16 M and N dimensions must be divisible by 128")
    if type(return_normal) is not bool or type(return_transposed) is not bool:
        raise TypeError("return_normal and return_transposed must be booleans")
    if not return_normal and not return_transposed:
        raise ValueError("at least one quantized layout must be requested")
    if x_bf16.dtype != torch.bfloat16 or not x_bf16.is_cuda:
        raise ValueError("x_bf16 must be a CUDA bfloat16 tensor")
    return _C.mxfp8_quantize(x_bf16, return_normal, return_transposed)


def _validate_fwd_bf16(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank,
                       schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
                       macrobatch_size, minibatch_size, *, combine_buffer=None, combine_buffer_ptrs=None,
                       w_shared_down=None, w_routed_down=None):
    T, H = _check_activation("x", x)
    I, E_l = _check_weights(w_shared_gate, w_routed_gate, H)
    _check_knobs(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptrs("x_ptrs", x_ptrs)
    if combine_buffer_ptrs is not None:
        _check_ptrs("combine_buffer_ptrs", combine_buffer_ptrs, ep_size)
    _check_schedule(schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, E_l)
    table = [
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (E_l, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (E_l, I, H)),
        ("schedule_peer_rank", schedule_peer_rank, None), ("schedule_peer_token_idx", schedule_peer_token_idx, None),
        ("num_tokens", num_tokens, None), ("tokens_per_expert", tokens_per_expert, None),
    ]
    if combine_buffer is not None:
        table += [("combine_buffer", combine_buffer, (T * topk, H)), ("w_shared_down", w_shared_down, (H, I)),
                  ("w_routed_down", w_routed_down, (E_l, H, I))]
    _check_shapes_devices(x.device, table)


@_op("mok::dispatch_mlp_swiglu_combine_fwd_bf16", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_bf16(
    x: torch.Tensor,
    x_ptrs: list[int],
    combine_buffer: torch.Tensor,
    combine_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
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
           torch.Tensor, torch.Tensor]:
    """Fused BF16 forward (reference: mok/ops.py:377-520).  Returns x_routed [MB,H], gate_shared [T,I],
    gate_routed [MB,I], up_shared, up_routed, hidden_shared, hidden_routed, y_shared [T,H], y_routed [MB,H];
    writes every peer's combine_buffer."""
    _validate_fwd_bf16(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank,
                       schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
                       macrobatch_size, minibatch_size, combine_buffer=combine_buffer,
                       combine_buffer_ptrs=combine_buffer_ptrs, w_shared_down=w_shared_down, w_routed_down=w_routed_down)
    return _C.dispatch_mlp_swiglu_combine_fwd_bf16(
        x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
        w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
        topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)


@_op("mok::recompute_forward_context_bf16", mutates_args=())
def recompute_forward_context_bf16(
    x: torch.Tensor,
    x_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Forward without the down projection and combine: rebuilds the saved context, bit-identical to
    the forward's (reference: mok/ops.py, recompute_forward_context_bf16; csrc/megakernel/recompute_forward_context.cuh)."""
    _validate_fwd_bf16(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank,
                       schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
                       macrobatch_size, minibatch_size)
    return _C.recompute_forward_context_bf16(
        x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank,
        schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
        minibatch_size)


@_op(
    "mok::dispatch_mlp_swiglu_combine_bwd_bf16",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed", "up_routed", "hidden_routed"),
)
def dispatch_mlp_swiglu_combine_bwd_bf16(
    d_y_buffer: torch.Tensor,
    d_y_buffer_ptrs: list[int],
    d_x_routed_buffer: torch.Tensor,
    d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: torch.Tensor,
    router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: torch.Tensor,
    d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
    x_routed: torch.Tensor,
    gate_shared: torch.Tensor,
    gate_routed: torch.Tensor,
    up_shared: torch.Tensor,
    up_routed: torch.Tensor,
    hidden_shared: torch.Tensor,
    hidden_routed: torch.Tensor,
    x: torch.Tensor,
    x_ptrs: list[int],
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
           torch.Tensor]:
    """Fused BF16 backward (reference: mok/ops.py:1079-1276).  Returns d_x_shared, d_x_routed, d_gate_shared,
    d_gate_routed, d_up_shared, d_up_routed, d_hidden_shared, d_hidden_routed, d_y_routed, d_w_shared_gate,
    d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down; writes every peer's
    d_x_routed_buffer and d_router_weight_buffer."""
    T, H = _check_activation("x", x)
    I, E_l = _check_weights(w_shared_gate, w_routed_gate, H)
    _check_knobs(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptrs("x_ptrs", x_ptrs)
    for name, ptrs in (("d_y_buffer_ptrs", d_y_buffer_ptrs), ("d_x_routed_buffer_ptrs", d_x_routed_buffer_ptrs),
                       ("router_weight_buffer_ptrs", router_weight_buffer_ptrs),
                       ("d_router_weight_buffer_ptrs", d_router_weight_buffer_ptrs)):
        _check_ptrs(name, ptrs, ep_size)
    _check_schedule(schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, E_l)
    MB = macrobatch_size
    _check_shapes_devices(x.device, [
        ("d_y_buffer", d_y_buffer, (T, H)), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H)),
        ("router_weight_buffer", router_weight_buffer, (T, topk)),
        ("d_router_weight_buffer", d_router_weight_buffer, (T, topk)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (E_l, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (E_l, I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (E_l, H, I)),
        ("x_routed", x_routed, (MB, H)), ("gate_shared", gate_shared, (T, I)), ("gate_routed", gate_routed, (MB, I)),
        ("up_shared", up_shared, (T, I)), ("up_routed", up_routed, (MB, I)),
        ("hidden_shared", hidden_shared, (T, I)), ("hidden_routed", hidden_routed, (MB, I)),
        ("schedule_peer_rank", schedule_peer_rank, None), ("schedule_peer_token_idx", schedule_peer_token_idx, None),
        ("num_tokens", num_tokens, None), ("tokens_per_expert", tokens_per_expert, None),
    ])
    return _C.dispatch_mlp_swiglu_combine_bwd_bf16(
        d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
        router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate,
        w_shared_up, w_routed_up, w_shared_down, w_routed_down, x_routed, gate_shared, gate_routed, up_shared,
        up_routed, hidden_shared, hidden_routed, x, x_ptrs, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
        tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)


@_op("mok::fwd_epilogue", mutates_args=())
def fwd_epilogue(y_shared: torch.Tensor, combine_buffer: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
    """output = y_shared + sum_k topk_weights[:, k] * combine_buffer[t*K+k] (reference: mok/ops.py:1279-1313)."""
    T, H = _check_activation("y_shared", y_shared)
    if topk_weights.device != y_shared.device or combine_buffer.device != y_shared.device:
        raise ValueError("all tensors must be on the same CUDA device")
    if topk_weights.ndim != 2 or topk_weights.shape[0] != T:
        raise ValueError("topk_weights must have shape (num_local_tokens, topk)")
    K = topk_weights.shape[1]
    if not 0 < K <= 255:
        raise ValueError("topk must be in [1, 255]")
    if tuple(combine_buffer.shape) != (T * K, H):
        raise ValueError("combine_buffer must have shape (num_local_tokens * topk, hidden_size)")
    return _C.fwd_epilogue(y_shared, combine_buffer, topk_weights)


@_op("mok::bwd_epilogue", mutates_args=())
def bwd_epilogue(d_x_shared: torch.Tensor, d_x_routed_buffer: torch.Tensor) -> torch.Tensor:
    """d_x = d_x_shared + sum_k d_x_routed_buffer[t*K+k] (reference: mok/ops.py:1316-1349)."""
    T, H = _check_activation("d_x_shared", d_x_shared)
    if d_x_routed_buffer.device != d_x_shared.device:
        raise ValueError("d_x_routed_buffer must be on the same CUDA device")
    if (d_x_routed_buffer.ndim != 2 or d_x_routed_buffer.shape[1] != H or d_x_routed_buffer.shape[0] % T != 0
            or d_x_routed_buffer.shape[0] == 0 or d_x_routed_buffer.shape[0] > T * 255):
        raise ValueError("d_x_routed_buffer must have shape (num_local_tokens * topk, hidden_size)")
    return _C.bwd_epilogue(d_x_shared, d_x_routed_buffer)


_fake_impls.register()

# the MXFP8 layer operators live in their own module; `mok.ops` is the one public namespace
from .ops_mxfp8 import (  # noqa: E402,F401
    dispatch_mlp_swiglu_combine_bwd_mxfp8,
    dispatch_mlp_swiglu_combine_fwd_mxfp8,
    recompute_forward_context_mxfp8,
)
