"""`mok.functional`: configuration, symmetric workspace, schedule building and the
forward / backward / recompute calls of the MoE layer -- the functional surface of
the reference (mok/functional.py there: MoKConfig :24-31, MoKWorkspace :53-88,
create_workspace :162, get_workspace :279, build_schedule :349, forward :470,
recompute_forward_context :571, backward :652), with the same names, argument
order, return values and exceptions.

The workspace is six symmetric buffers per rank plus a route-gather buffer and a
barrier word.  With ep_size == 1 they are ordinary device tensors; otherwise they
come from torch's symmetric memory, whose rendezvous yields every peer's unicast
address.  NCCL is used for that bootstrap only: the data path is peer loads and
stores issued by this library's kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from . import ops

MAX_EP = ops.MAX_EP


@dataclass(frozen=True, slots=True)
class MoKConfig:
    fwd_num_comm_sms: int = 40
    bwd_num_comm_sms: int = 28
    minibatch_size: int = 4096
    macrobatch_size: int = 131072
    schedule_capacity_multiplier: float = 0.5
    all_gather_top_experts_chunk_bytes: int = 2048


@dataclass(frozen=True, slots=True)
class MoKSchedule:
    peer_rank: torch.Tensor          # (schedule_capacity,) int32
    peer_token_idx: torch.Tensor     # (schedule_capacity,) int32
    num_tokens: torch.Tensor         # (1,) int32
    tokens_per_expert: torch.Tensor  # (num_local_experts,) int32


@dataclass(frozen=True, slots=True)
class MoKForwardContext:
    x_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    gate_shared: torch.Tensor
    gate_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    up_shared: torch.Tensor
    up_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    hidden_shared: torch.Tensor
    hidden_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]


@dataclass(slots=True)
class MoKWorkspace:
    group_name: str
    ep_rank: int
    ep_size: int
    device: torch.device
    num_local_tokens: int
    hidden_size: int
    topk: int
    schedule_capacity: int
    x_buffer: torch.Tensor                       # (T, H) bf16
    x_buffer_handle: Any
    x_buffer_ptrs: list[int]
    combine_buffer: torch.Tensor                 # (T*K, H) bf16
    combine_buffer_handle: Any
    combine_buffer_ptrs: list[int]
    d_y_buffer: torch.Tensor                     # (T, H) bf16
    d_y_buffer_handle: Any
    d_y_buffer_ptrs: list[int]
    d_x_routed_buffer: torch.Tensor              # (T*K, H) bf16
    d_x_routed_buffer_handle: Any
    d_x_routed_buffer_ptrs: list[int]
    router_weight_buffer: torch.Tensor           # (T, K) f32
    router_weight_buffer_handle: Any
    router_weight_buffer_ptrs: list[int]
    d_router_weight_buffer: torch.Tensor         # (T, K) f32
    d_router_weight_buffer_handle: Any
    d_router_weight_buffer_ptrs: list[int]
    all_gather_top_experts_buffer: torch.Tensor  # (ep_size, T, K) int32
    all_gather_top_experts_buffer_handle: Any
    all_gather_top_experts_buffer_multicast_ptr: int
    barrier_buffer: torch.Tensor                 # (1,) int32
    barrier_buffer_handle: Any
    barrier_buffer_ptrs: list[int]
    barrier_buffer_multicast_ptr: int
    barrier_target: torch.Tensor                 # (1,) int32
    all_gather_top_experts_buffer_ptrs: list[int] | None = None   # peers' unicast addresses (not in the reference)


_WORKSPACE_CACHE: dict[tuple[str, int, int, int, int, int], MoKWorkspace] = {}


def schedule_capacity_factor(config: MoKConfig, ep_size: int) -> int:
    """schedule_capacity = T * K * max(2, ceil(ep_size * multiplier)) (reference: mok/functional.py:198,209)."""
    return max(2, math.ceil(ep_size * config.schedule_capacity_multiplier))


def validate_workspace_args(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device,
                            num_local_tokens: int, hidden_size: int, topk: int) -> None:
    """Argument checks shared by create_workspace and get_workspace (reference: mok/functional.py:94-159)."""
    m = config.schedule_capacity_multiplier
    if type(m) not in (int, float) or not math.isfinite(m) or m <= 0:
        raise ValueError("schedule_capacity_multiplier must be a positive finite number")
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized")
    if not isinstance(group, dist.ProcessGroup):
        raise TypeError("group must be a torch.distributed.ProcessGroup")
    if not isinstance(device, torch.device):
        raise TypeError("device must be a torch.device")
    if device.type != "cuda":
        raise ValueError("device must be a CUDA device")
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index != torch.cuda.current_device():
        raise ValueError("MoK workspace device must be the current CUDA device")
    if torch.cuda.get_device_capability(index) not in ((10, 0), (10, 3)):
        raise NotImplementedError("MoK currently requires an SM100 or SM103 GPU")
    validate_shape_args(num_local_tokens, hidden_size, topk)
    name = group.group_name
    if not isinstance(name, str) or not name:
        raise RuntimeError("process group must have a nonempty group_name")
    ep_rank, ep_size = dist.get_rank(group=group), dist.get_world_size(group=group)
    if not 1 <= ep_size <= MAX_EP:
        raise ValueError(f"MoK EP size must be in [1, {MAX_EP}]")
    if not 0 <= ep_rank < ep_size:
        raise RuntimeError("current process is not a member of the EP process group")


def validate_shape_args(num_local_tokens: int, hidden_size: int, topk: int) -> None:
    if type(num_local_tokens) is not int or num_local_tokens < 512:
        raise ValueError("num_local_tokens must be an integer at least 512")
    if num_local_tokens % 256 != 0:
        raise ValueError("num_local_tokens must be divisible by 256")
    if type(hidden_size) is not int or hidden_size <= 0:
        raise ValueError("hidden_size must be a positive integer")
    if hidden_size % 256 != 0:
        raise ValueError("hidden_size must be divisible by 256")
    if type(topk) is not int or not 0 < topk <= 255:
        raise ValueError("topk must be an integer in [1, 255]")


def check_identical_shapes(group: dist.ProcessGroup, device: torch.device, num_local_tokens: int, hidden_size: int,
                           topk: int) -> None:
    """All EP ranks must use the same (T, H, K); one-time collective with a host read
    (reference: mok/functional.py:200-205).  Works on any backend/device."""
    ep_size = dist.get_world_size(group=group)
    local = torch.tensor([num_local_tokens, hidden_size, topk], dtype=torch.int64, device=device)
    gathered = torch.empty(ep_size * 3, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, local, group=group)
    if not torch.all(gathered.view(ep_size, 3) == local).item():
        raise ValueError("MoK requires identical token, hidden, and top-k shapes on every EP rank")


def create_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                     hidden_size: int, topk: int) -> MoKWorkspace:
    """Creates a new caller-owned workspace (reference: mok/functional.py:162-276)."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens,
                            hidden_size=hidden_size, topk=topk)
    index = device.index if device.index is not None else torch.cuda.current_device()
    device = torch.device("cuda", index)
    group_name = group.group_name
    ep_rank, ep_size = dist.get_rank(group=group), dist.get_world_size(group=group)
    check_identical_shapes(group, device, num_local_tokens, hidden_size, topk)
    capacity = num_local_tokens * topk * schedule_capacity_factor(config, ep_size)

    symm_mem = None
    if ep_size > 1:
        import torch.distributed._symmetric_memory as symm_mem
        symm_mem.enable_symm_mem_for_group(group_name)

    def allocate(*shape: int, dtype: torch.dtype, zero: bool = False):
        if ep_size == 1:
            buf = (torch.zeros if zero else torch.empty)(*shape, dtype=dtype, device=device)
            return buf, None, [int(buf.data_ptr())]
        buf = symm_mem.empty(*shape, dtype=dtype, device=device)
        if zero:
            buf.zero_()
        handle = symm_mem.rendezvous(buf, group_name)
        return buf, handle, [int(handle.buffer_ptrs[r]) for r in range(ep_size)]

    T, H, K = num_local_tokens, hidden_size, topk
    x, xh, xp = allocate(T, H, dtype=torch.bfloat16)
    cb, cbh, cbp = allocate(T * K, H, dtype=torch.bfloat16)
    dy, dyh, dyp = allocate(T, H, dtype=torch.bfloat16)
    dx, dxh, dxp = allocate(T * K, H, dtype=torch.bfloat16)
    rw, rwh, rwp = allocate(T, K, dtype=torch.float32)
    drw, drwh, drwp = allocate(T, K, dtype=torch.float32)
    ag, agh, agp = allocate(ep_size, T, K, dtype=torch.int32)
    bar, barh, barp = allocate(1, dtype=torch.int32, zero=True)
    target = torch.zeros(1, dtype=torch.int32, device=device)
    dist.barrier(group=group, async_op=True, device_ids=[index]).block_current_stream()
    torch.cuda.current_stream().synchronize()   # the zeroed barrier word must be visible before any peer signals it

    return MoKWorkspace(
        group_name=group_name, ep_rank=ep_rank, ep_size=ep_size, device=device, num_local_tokens=T, hidden_size=H,
        topk=K, schedule_capacity=capacity,
        x_buffer=x, x_buffer_handle=xh, x_buffer_ptrs=xp,
        combine_buffer=cb, combine_buffer_handle=cbh, combine_buffer_ptrs=cbp,
        d_y_buffer=dy, d_y_buffer_handle=dyh, d_y_buffer_ptrs=dyp,
        d_x_routed_buffer=dx, d_x_routed_buffer_handle=dxh, d_x_routed_buffer_ptrs=dxp,
        router_weight_buffer=rw, router_weight_buffer_handle=rwh, router_weight_buffer_ptrs=rwp,
        d_router_weight_buffer=drw, d_router_weight_buffer_handle=drwh, d_router_weight_buffer_ptrs=drwp,
        all_gather_top_experts_buffer=ag, all_gather_top_experts_buffer_handle=agh,
        all_gather_top_experts_buffer_multicast_ptr=int(ag.data_ptr()),
        barrier_buffer=bar, barrier_buffer_handle=barh, barrier_buffer_ptrs=barp,
        barrier_buffer_multicast_ptr=int(bar.data_ptr()), barrier_target=target,
        all_gather_top_experts_buffer_ptrs=agp,
    )


def get_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                  hidden_size: int, topk: int) -> MoKWorkspace:
    """Returns a cached workspace, creating one if absent (reference: mok/functional.py:279-330)."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens,
                            hidden_size=hidden_size, topk=topk)
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (group.group_name, index, num_local_tokens, hidden_size, topk,
           schedule_capacity_factor(config, dist.get_world_size(group=group)))
    ws = _WORKSPACE_CACHE.get(key)
    if ws is None:
        ws = create_workspace(config, group, device=torch.device("cuda", index), num_local_tokens=num_local_tokens,
                              hidden_size=hidden_size, topk=topk)
        _WORKSPACE_CACHE[key] = ws
    return ws


def clear_workspace_cache() -> None:
    """Clears cached workspaces after all participating ranks synchronize (reference: mok/functional.py:333-346)."""
    for ws in _WORKSPACE_CACHE.values():
        _barrier(ws)
        torch.cuda.synchronize(ws.device)
    _WORKSPACE_CACHE.clear()


def _barrier(ws: MoKWorkspace) -> None:
    ops.call(ops.barrier_all, ws.barrier_buffer, ws.barrier_buffer_ptrs, ws.barrier_buffer_multicast_ptr,
             ws.barrier_target)


def validate_config(config: MoKConfig, num_sms: int, route_buffer_bytes: int, smem_optin: int = 232448) -> None:
    """Checks of build_schedule on the six knobs (reference: mok/functional.py:367-398)."""
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    for name in ("fwd_num_comm_sms", "bwd_num_comm_sms"):
        v = getattr(config, name)
        if type(v) is not int or v <= 0:
            raise ValueError(f"{name} must be a positive integer")
        if v % 2 != 0:
            raise ValueError(f"{name} must be even")
    if config.fwd_num_comm_sms >= num_sms or config.bwd_num_comm_sms >= num_sms:
        raise ValueError("communication-SM counts must leave at least one compute SM")
    mb, MB = config.minibatch_size, config.macrobatch_size
    if type(mb) is not int or mb <= 0 or mb % 256 != 0:
        raise ValueError("minibatch_size must be positive and divisible by 256")
    if type(MB) is not int or MB <= 0 or MB % mb != 0:
        raise ValueError("macrobatch_size must be a positive multiple of minibatch_size")
    cb = config.all_gather_top_experts_chunk_bytes
    if type(cb) is not int or cb <= 0 or cb % 16 != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must be a positive multiple of 16")
    if cb + 1024 > smem_optin:
        raise ValueError("all_gather_top_experts_chunk_bytes exceeds device dynamic shared-memory capacity")
    if route_buffer_bytes % cb != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must divide one rank's route-buffer bytes")


def build_schedule(workspace: MoKWorkspace, config: MoKConfig, top_experts: torch.Tensor, *,
                   num_local_experts: int) -> MoKSchedule:
    """All-gathers routing choices and builds this rank's padded expert schedule
    (reference: mok/functional.py:349-425)."""
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    props = torch.cuda.get_device_properties(workspace.device)
    validate_config(config, props.multi_processor_count, workspace.num_local_tokens * workspace.topk * 4,
                    props.shared_memory_per_block_optin)
    if not top_experts.is_cuda or top_experts.device != workspace.device:
        raise ValueError("top_experts must be on the workspace CUDA device")
    if top_experts.dtype != torch.int64:
        raise TypeError("top_experts must have dtype torch.int64")
    if not top_experts.is_contiguous():
        raise ValueError("top_experts must be contiguous")
    if tuple(top_experts.shape) != (workspace.num_local_tokens, workspace.topk):
        raise ValueError("top_experts must have shape (num_local_tokens, topk)")
    if type(num_local_experts) is not int or num_local_experts <= 0:
        raise ValueError("num_local_experts must be a positive integer")

    ops.call(
        ops.all_gather_top_experts, top_experts.to(torch.int32), workspace.all_gather_top_experts_buffer,
        workspace.all_gather_top_experts_buffer_multicast_ptr, workspace.ep_rank,
        config.all_gather_top_experts_chunk_bytes, workspace.all_gather_top_experts_buffer_ptrs)
    _barrier(workspace)
    peer_rank, peer_token_idx, num_tokens, tokens_per_expert = ops.call(
        ops.schedule, workspace.all_gather_top_experts_buffer, num_local_experts, workspace.schedule_capacity,
        workspace.ep_rank)
    return MoKSchedule(peer_rank=peer_rank, peer_token_idx=peer_token_idx, num_tokens=num_tokens,
                       tokens_per_expert=tokens_per_expert)


def validate_inputs(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
                    router_weights: torch.Tensor | None = None, grad_output: torch.Tensor | None = None) -> None:
    """Runtime inputs against the workspace and schedule (reference: mok/functional.py:428-467)."""
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(schedule, MoKSchedule):
        raise TypeError("schedule must be a MoKSchedule")
    act = (workspace.num_local_tokens, workspace.hidden_size)
    tensors = [("x", x, torch.bfloat16, act)]
    if grad_output is not None:
        tensors.append(("grad_output", grad_output, torch.bfloat16, act))
    if router_weights is not None:
        tensors.append(("router_weights", router_weights, torch.float32, (workspace.num_local_tokens, workspace.topk)))
    for name, t, dtype, shape in tensors:
        if not t.is_cuda or t.device != workspace.device or t.dtype != dtype or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} on the workspace CUDA device")
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} shape does not match the workspace")
    if schedule.peer_rank.numel() != workspace.schedule_capacity:
        raise ValueError("schedule capacity does not match the workspace")


def _is_mxfp8(weights) -> bool:
    return isinstance(weights, tuple)


def _stage(buffer: torch.Tensor, value: torch.Tensor) -> None:
    """Copies `value` into the workspace's symmetric `buffer` (reference: mok/functional.py:509-510, 709-711, each
    marked there as removable).  A caller that produced the value in the buffer itself (it passes `workspace.x_buffer`,
    `workspace.d_y_buffer` or `workspace.router_weight_buffer` as the argument) pays no copy."""
    if value is buffer:
        return
    if not torch.compiler.is_compiling() and not isinstance(value, torch._subclasses.FakeTensor):
        if value.data_ptr() == buffer.data_ptr() and value.shape == buffer.shape and value.stride() == buffer.stride():
            return
    buffer.copy_(value)


def forward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
            router_weights: torch.Tensor, shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor,
            shared_down_weights: torch.Tensor, routed_gate_weights, routed_up_weights, routed_down_weights,
            swiglu_limit: float | None = None) -> tuple[torch.Tensor, MoKForwardContext]:
    """Runs the MoE forward pass (reference: mok/functional.py:470-568).  Routed weights are bf16 tensors
    [E_l, I, H] / [E_l, H, I], or (fp8, scales) pairs for MXFP8."""
    validate_inputs(config, workspace, schedule, x, router_weights)
    ws = workspace
    _stage(ws.x_buffer, x)
    _stage(ws.router_weight_buffer, router_weights)
    _barrier(ws)
    if _is_mxfp8(routed_gate_weights):
        from . import ops_mxfp8
        (gq, gs), (uq, us), (dq, ds) = routed_gate_weights, routed_up_weights, routed_down_weights
        (x_fp8_t, x_sc_t, gate_shared, gate_fp8, gate_sc, up_shared, up_fp8, up_sc, hidden_shared, hidden_fp8_t,
         hidden_sc_t, y_shared, _y_routed) = ops.call(
            ops_mxfp8.dispatch_mlp_swiglu_combine_fwd_mxfp8,
            ws.x_buffer, ws.x_buffer_ptrs, ws.combine_buffer, ws.combine_buffer_ptrs,
            shared_gate_weights, gq, gs, shared_up_weights, uq, us, shared_down_weights, dq, ds,
            schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert,
            ws.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
        ctx = MoKForwardContext(x_routed=(x_fp8_t, x_sc_t), gate_shared=gate_shared, gate_routed=(gate_fp8, gate_sc),
                                up_shared=up_shared, up_routed=(up_fp8, up_sc), hidden_shared=hidden_shared,
                                hidden_routed=(hidden_fp8_t, hidden_sc_t))
    else:
        (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed, y_shared,
         _y_routed) = ops.call(
            ops.dispatch_mlp_swiglu_combine_fwd_bf16,
            ws.x_buffer, ws.x_buffer_ptrs, ws.combine_buffer, ws.combine_buffer_ptrs,
            shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights,
            schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert,
            ws.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
        ctx = MoKForwardContext(x_routed=x_routed, gate_shared=gate_shared, gate_routed=gate_routed,
                                up_shared=up_shared, up_routed=up_routed, hidden_shared=hidden_shared,
                                hidden_routed=hidden_routed)
    _barrier(ws)
    output = ops.call(ops.fwd_epilogue, y_shared, ws.combine_buffer, ws.router_weight_buffer)
    return output, ctx


def recompute_forward_context(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
                              shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor,
                              routed_gate_weights, routed_up_weights,
                              swiglu_limit: float | None = None) -> MoKForwardContext:
    """Recomputes the intermediates the backward pass needs (reference: mok/functional.py:571-649)."""
    validate_inputs(config, workspace, schedule, x)
    if _is_mxfp8(routed_gate_weights) != _is_mxfp8(routed_up_weights):
        raise TypeError("routed gate and up weights must use the same precision representation")
    if _is_mxfp8(routed_gate_weights) and (len(routed_gate_weights) != 2 or len(routed_up_weights) != 2):
        raise ValueError("MXFP8 routed gate and up weights must be data/scale pairs")
    ws = workspace
    _stage(ws.x_buffer, x)
    _barrier(ws)
    if _is_mxfp8(routed_gate_weights):
        from . import ops_mxfp8
        (gq, gs), (uq, us) = routed_gate_weights, routed_up_weights
        (x_fp8_t, x_sc_t, gate_shared, gate_fp8, gate_sc, up_shared, up_fp8, up_sc, hidden_shared, hidden_fp8_t,
         hidden_sc_t) = ops.call(
            ops_mxfp8.recompute_forward_context_mxfp8,
            ws.x_buffer, ws.x_buffer_ptrs, shared_gate_weights, gq, gs, shared_up_weights, uq, us,
            schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert,
            ws.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
        ctx = MoKForwardContext(x_routed=(x_fp8_t, x_sc_t), gate_shared=gate_shared, gate_routed=(gate_fp8, gate_sc),
                                up_shared=up_shared, up_routed=(up_fp8, up_sc), hidden_shared=hidden_shared,
                                hidden_routed=(hidden_fp8_t, hidden_sc_t))
    else:
        (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared,
         hidden_routed) = ops.call(
            ops.recompute_forward_context_bf16,
            ws.x_buffer, ws.x_buffer_ptrs, shared_gate_weights, routed_gate_weights, shared_up_weights,
            routed_up_weights, schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens,
            schedule.tokens_per_expert, ws.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size,
            config.minibatch_size)
        ctx = MoKForwardContext(x_routed=x_routed, gate_shared=gate_shared, gate_routed=gate_routed,
                                up_shared=up_shared, up_routed=up_routed, hidden_shared=hidden_shared,
                                hidden_routed=hidden_routed)
    _barrier(ws)
    return ctx


def backward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, forward_context: MoKForwardContext,
             grad_output: torch.Tensor, x: torch.Tensor, router_weights: torch.Tensor,
             shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor, shared_down_weights: torch.Tensor,
             routed_gate_weights, routed_up_weights, routed_down_weights, swiglu_limit: float | None = None):
    """Runs the MoE backward pass (reference: mok/functional.py:652-780).  Returns (d_x, d_router_weights,
    d_routed_gate_weights, d_routed_up_weights, d_routed_down_weights, d_shared_gate_weights,
    d_shared_up_weights, d_shared_down_weights)."""
    validate_inputs(config, workspace, schedule, x, router_weights, grad_output)
    if not isinstance(forward_context, MoKForwardContext):
        raise TypeError("forward_context must be a MoKForwardContext")
    ws = workspace
    _stage(ws.d_y_buffer, grad_output)
    _stage(ws.x_buffer, x)
    _stage(ws.router_weight_buffer, router_weights)
    _barrier(ws)
    ctx = forward_context
    if _is_mxfp8(routed_gate_weights):
        from . import ops_mxfp8
        gq, gs, gtq, gts = routed_gate_weights
        uq, us, utq, uts = routed_up_weights
        dtq, dts = routed_down_weights
        outs = ops.call(
            ops_mxfp8.dispatch_mlp_swiglu_combine_bwd_mxfp8,
            ws.d_y_buffer, ws.d_y_buffer_ptrs, ws.d_x_routed_buffer, ws.d_x_routed_buffer_ptrs,
            ws.router_weight_buffer, ws.router_weight_buffer_ptrs, ws.d_router_weight_buffer,
            ws.d_router_weight_buffer_ptrs,
            shared_gate_weights, gtq, gts, shared_up_weights, utq, uts, shared_down_weights, dtq, dts,
            ctx.x_routed[0], ctx.x_routed[1], ctx.gate_shared, ctx.gate_routed[0], ctx.gate_routed[1],
            ctx.up_shared, ctx.up_routed[0], ctx.up_routed[1], ctx.hidden_shared, ctx.hidden_routed[0],
            ctx.hidden_routed[1], ws.x_buffer, ws.x_buffer_ptrs, gq, gs, uq, us,
            schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert,
            ws.topk, swiglu_limit, config.bwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
        d_x_shared = outs[0]
        d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down = outs[-6:]
    else:
        outs = ops.call(
            ops.dispatch_mlp_swiglu_combine_bwd_bf16,
            ws.d_y_buffer, ws.d_y_buffer_ptrs, ws.d_x_routed_buffer, ws.d_x_routed_buffer_ptrs,
            ws.router_weight_buffer, ws.router_weight_buffer_ptrs, ws.d_router_weight_buffer,
            ws.d_router_weight_buffer_ptrs,
            shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights,
            ctx.x_routed, ctx.gate_shared, ctx.gate_routed, ctx.up_shared, ctx.up_routed, ctx.hidden_shared,
            ctx.hidden_routed, ws.x_buffer, ws.x_buffer_ptrs,
            schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert,
            ws.topk, swiglu_limit, config.bwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
        d_x_shared = outs[0]
        d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down = outs[-6:]
    _barrier(ws)
    d_x = ops.call(ops.bwd_epilogue, d_x_shared, ws.d_x_routed_buffer)
    d_router_weights = ws.d_router_weight_buffer.clone()
    return (d_x, d_router_weights, d_w_routed_gate, d_w_routed_up, d_w_routed_down,
            d_w_shared_gate, d_w_shared_up, d_w_shared_down)
