"""ctypes binding of the MXFP8 layer entry points of libmok_b200.so: the three `*_mxfp8`
functions of the reference's `_C` module (csrc/bindings.cu:19-48, 77-85 there).  Allocates the
outputs the reference allocates plus the work buffers the C-ABI asks the caller for."""
from __future__ import annotations

import ctypes

import torch

from . import _C
from ._C import c_f32, c_int, c_u64p, c_vp, _ck, _p, _ptr_array, _stream, lib

_SIZES = ["ep_size", "ep_rank", "num_local_tokens", "hidden", "intermediate", "num_local_experts", "topk",
          "schedule_capacity", "macrobatch_size", "minibatch_size", "num_comm_sms", "has_swiglu_limit"]
_SCHED = ["peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"]


class FwdMxfp8Args(ctypes.Structure):
    _fields_ = (
        [(n, c_int) for n in _SIZES] + [("swiglu_limit", c_f32)] + [(n, c_vp) for n in _SCHED]
        + [("x_ptrs_host", c_u64p), ("combine_ptrs_host", c_u64p)]
        + [(n, c_vp) for n in (
            "w_shared_gate", "w_shared_up", "w_shared_down",
            "w_routed_gate", "w_routed_gate_sc", "w_routed_up", "w_routed_up_sc", "w_routed_down", "w_routed_down_sc",
            "x_fp8_t", "x_sc_t", "gate_shared", "up_shared", "hidden_shared", "gate_fp8", "gate_sc", "up_fp8", "up_sc",
            "hidden_fp8_t", "hidden_sc_t", "y_shared", "y_routed",
            "x_routed", "x_fp8", "x_sc", "hidden_fp8", "hidden_sc", "scratch", "status")]
        + [("skip_down_combine", c_int)])


class BwdMxfp8Args(ctypes.Structure):
    _fields_ = (
        [(n, c_int) for n in _SIZES] + [("swiglu_limit", c_f32)] + [(n, c_vp) for n in _SCHED]
        + [(n, c_u64p) for n in ("d_y_ptrs_host", "d_x_routed_ptrs_host", "router_weight_ptrs_host",
                                 "d_router_weight_ptrs_host", "x_ptrs_host")]
        + [(n, c_vp) for n in (
            "w_shared_gate", "w_shared_up", "w_shared_down",
            "w_routed_gate_t", "w_routed_gate_t_sc", "w_routed_up_t", "w_routed_up_t_sc", "w_routed_down_t", "w_routed_down_t_sc",
            "x_fp8_t", "x_sc_t", "gate_shared", "gate_fp8", "gate_sc", "up_shared", "up_fp8", "up_sc",
            "hidden_shared", "hidden_fp8_t", "hidden_sc_t",
            "d_x_shared", "d_x_routed", "d_gate_shared", "d_gate_fp8", "d_gate_sc", "d_up_shared", "d_up_fp8", "d_up_sc",
            "d_hidden_shared", "d_hidden_routed", "d_y_fp8", "d_y_sc",
            "d_w_shared_gate", "d_w_routed_gate", "d_w_shared_up", "d_w_routed_up", "d_w_shared_down", "d_w_routed_down",
            "d_y_routed", "d_y_fp8_t", "d_y_sc_t", "d_gate_fp8_t", "d_gate_sc_t", "d_up_fp8_t", "d_up_sc_t", "partials",
            "w_routed_gate", "w_routed_gate_sc", "w_routed_up", "w_routed_up_sc",
            "x_routed", "x_fp8", "x_sc", "hidden_fp8", "hidden_sc",
            "scratch", "status")])


lib.mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8.restype = c_int
lib.mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8.argtypes = [ctypes.POINTER(FwdMxfp8Args), c_vp]
lib.mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8.restype = c_int
lib.mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8.argtypes = [ctypes.POINTER(BwdMxfp8Args), c_vp]
lib.mokb_struct_sizes_mxfp8.restype = c_int
lib.mokb_struct_sizes_mxfp8.argtypes = [ctypes.POINTER(c_int), c_int]

_sizes = (c_int * 3)()
lib.mokb_struct_sizes_mxfp8(_sizes, 3)
_mine = (ctypes.sizeof(FwdMxfp8Args), ctypes.sizeof(BwdMxfp8Args), ctypes.sizeof(_C.GemmFp8Args))
if tuple(_sizes) != _mine:
    raise ImportError(f"MXFP8 struct layout mismatch: library {tuple(_sizes)}, binding {_mine}")

EXPORTED = ["mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8", "mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8",
            "mokb_struct_sizes_mxfp8"]

F8 = torch.float8_e4m3fn


def _q(rows, cols, dev):
    """E4M3 [rows, cols] + packed scales."""
    return (torch.empty(rows, cols, dtype=F8, device=dev),
            torch.empty(rows // 128, cols // 128, 32, 16, dtype=torch.uint8, device=dev))


def _fwd(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up,
         w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc, schedule_peer_rank,
         schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
         minibatch_size, skip):
    a = FwdMxfp8Args()
    T, H, I, E_l, dev, scratch = _C._common(
        a, x_ptrs=x_ptrs, x_like=x, w_shared_gate=w_shared_gate, w_routed_gate=w_routed_gate,
        schedule_peer_rank=schedule_peer_rank, schedule_peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
        tokens_per_expert=tokens_per_expert, topk=topk, swiglu_limit=swiglu_limit, num_comm_sms=num_comm_sms,
        macrobatch_size=macrobatch_size, minibatch_size=minibatch_size)
    MB = macrobatch_size
    bf = dict(dtype=torch.bfloat16, device=dev)
    keep = [_ptr_array(x_ptrs)]
    a.x_ptrs_host = keep[0]
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = _p(w_shared_gate), _p(w_shared_up), _p(w_shared_down)
    a.w_routed_gate, a.w_routed_gate_sc = _p(w_routed_gate), _p(w_routed_gate_sc)
    a.w_routed_up, a.w_routed_up_sc = _p(w_routed_up), _p(w_routed_up_sc)
    a.w_routed_down, a.w_routed_down_sc = _p(w_routed_down), _p(w_routed_down_sc)
    x_fp8_t, x_sc_t = _q(H, MB, dev)
    gate_shared, up_shared, hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    gate_fp8, gate_sc = _q(MB, I, dev)
    up_fp8, up_sc = _q(MB, I, dev)
    hidden_fp8_t, hidden_sc_t = _q(I, MB, dev)
    y_shared = y_routed = None
    if not skip:
        y_shared, y_routed = torch.empty(T, H, **bf), torch.empty(MB, H, **bf)
        keep.append(_ptr_array(combine_buffer_ptrs))
        a.combine_ptrs_host = keep[1]
    work = [torch.empty(MB, H, **bf), *_q(MB, H, dev), *_q(MB, I, dev)]
    (a.x_fp8_t, a.x_sc_t, a.gate_shared, a.up_shared, a.hidden_shared, a.gate_fp8, a.gate_sc, a.up_fp8, a.up_sc,
     a.hidden_fp8_t, a.hidden_sc_t, a.y_shared, a.y_routed) = map(_p, (
        x_fp8_t, x_sc_t, gate_shared, up_shared, hidden_shared, gate_fp8, gate_sc, up_fp8, up_sc, hidden_fp8_t,
        hidden_sc_t, y_shared, y_routed if _C.KEEP_STAGING_ROWS else None))      # staging rows: see _C.KEEP_STAGING_ROWS
    (a.x_routed, a.x_fp8, a.x_sc, a.hidden_fp8, a.hidden_sc) = map(_p, work)
    a.skip_down_combine = 1 if skip else 0
    _ck(lib.mokb_dispatch_mlp_swiglu_combine_fwd_mxfp8(ctypes.byref(a), _stream()))
    return (x_fp8_t, x_sc_t, gate_shared, gate_fp8, gate_sc, up_shared, up_fp8, up_sc, hidden_shared, hidden_fp8_t,
            hidden_sc_t, y_shared, y_routed)


def dispatch_mlp_swiglu_combine_fwd_mxfp8(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate,
                                          w_routed_gate_sc, w_shared_up, w_routed_up, w_routed_up_sc, w_shared_down,
                                          w_routed_down, w_routed_down_sc, schedule_peer_rank, schedule_peer_token_idx,
                                          num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
                                          macrobatch_size, minibatch_size):
    return _fwd(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc,
                w_shared_up, w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc,
                schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                num_comm_sms, macrobatch_size, minibatch_size, False)


def recompute_forward_context_mxfp8(x, x_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up, w_routed_up,
                                    w_routed_up_sc, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
                                    tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
    return _fwd(x, x_ptrs, None, None, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up, w_routed_up,
                w_routed_up_sc, None, None, None, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
                tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, True)[:11]


def dispatch_mlp_swiglu_combine_bwd_mxfp8(
        d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
        router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs,
        w_shared_gate, w_routed_gate_T, w_routed_gate_T_sc, w_shared_up, w_routed_up_T, w_routed_up_T_sc,
        w_shared_down, w_routed_down_T, w_routed_down_T_sc,
        x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared, up_fp8_routed,
        up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed, x, x_ptrs,
        w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc,
        schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
        macrobatch_size, minibatch_size):
    a = BwdMxfp8Args()
    T, H, I, E_l, dev, scratch = _C._common(
        a, x_ptrs=x_ptrs, x_like=x, w_shared_gate=w_shared_gate, w_routed_gate=w_routed_gate,
        schedule_peer_rank=schedule_peer_rank, schedule_peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
        tokens_per_expert=tokens_per_expert, topk=topk, swiglu_limit=swiglu_limit, num_comm_sms=num_comm_sms,
        macrobatch_size=macrobatch_size, minibatch_size=minibatch_size)
    MB = macrobatch_size
    bf = dict(dtype=torch.bfloat16, device=dev)
    keep = [_ptr_array(p) for p in (d_y_buffer_ptrs, d_x_routed_buffer_ptrs, router_weight_buffer_ptrs,
                                    d_router_weight_buffer_ptrs, x_ptrs)]
    (a.d_y_ptrs_host, a.d_x_routed_ptrs_host, a.router_weight_ptrs_host, a.d_router_weight_ptrs_host,
     a.x_ptrs_host) = keep
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = _p(w_shared_gate), _p(w_shared_up), _p(w_shared_down)
    a.w_routed_gate_t, a.w_routed_gate_t_sc = _p(w_routed_gate_T), _p(w_routed_gate_T_sc)
    a.w_routed_up_t, a.w_routed_up_t_sc = _p(w_routed_up_T), _p(w_routed_up_T_sc)
    a.w_routed_down_t, a.w_routed_down_t_sc = _p(w_routed_down_T), _p(w_routed_down_T_sc)
    (a.x_fp8_t, a.x_sc_t, a.gate_shared, a.gate_fp8, a.gate_sc, a.up_shared, a.up_fp8, a.up_sc, a.hidden_shared,
     a.hidden_fp8_t, a.hidden_sc_t) = map(_p, (
        x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared, up_fp8_routed,
        up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed))
    d_x_shared, d_x_routed = torch.empty(T, H, **bf), torch.empty(MB, H, **bf)
    d_gate_shared, d_up_shared, d_hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    d_gate_fp8, d_gate_sc = _q(MB, I, dev)
    d_up_fp8, d_up_sc = _q(MB, I, dev)
    d_hidden_routed = torch.empty(MB, I, **bf)
    d_y_fp8, d_y_sc = _q(MB, H, dev)
    d_w_shared_gate, d_w_shared_up, d_w_shared_down = torch.empty(I, H, **bf), torch.empty(I, H, **bf), torch.empty(H, I, **bf)
    d_w_routed_gate, d_w_routed_up = torch.empty(E_l, I, H, **bf), torch.empty(E_l, I, H, **bf)
    d_w_routed_down = torch.empty(E_l, H, I, **bf)
    (a.d_x_shared, a.d_x_routed, a.d_gate_shared, a.d_gate_fp8, a.d_gate_sc, a.d_up_shared, a.d_up_fp8, a.d_up_sc,
     a.d_hidden_shared, a.d_hidden_routed, a.d_y_fp8, a.d_y_sc, a.d_w_shared_gate, a.d_w_routed_gate, a.d_w_shared_up,
     a.d_w_routed_up, a.d_w_shared_down, a.d_w_routed_down) = map(_p, (
        d_x_shared, d_x_routed if _C.KEEP_STAGING_ROWS else None, d_gate_shared, d_gate_fp8, d_gate_sc, d_up_shared, d_up_fp8,
        d_up_sc, d_hidden_shared, d_hidden_routed, d_y_fp8, d_y_sc, d_w_shared_gate, d_w_routed_gate, d_w_shared_up,
        d_w_routed_up, d_w_shared_down, d_w_routed_down))
    work = [torch.empty(MB, H, **bf), *_q(H, MB, dev), *_q(I, MB, dev), *_q(I, MB, dev),
            torch.empty(MB, I // 128, dtype=torch.float32, device=dev)]
    (a.d_y_routed, a.d_y_fp8_t, a.d_y_sc_t, a.d_gate_fp8_t, a.d_gate_sc_t, a.d_up_fp8_t, a.d_up_sc_t,
     a.partials) = map(_p, work)
    if a.schedule_capacity > MB:      # later macrobatches are replayed: forward weights and the forward's work buffers
        replay = [w_routed_gate, w_routed_gate_sc, w_routed_up, w_routed_up_sc, torch.empty(MB, H, **bf), *_q(MB, H, dev),
                  *_q(MB, I, dev)]
        (a.w_routed_gate, a.w_routed_gate_sc, a.w_routed_up, a.w_routed_up_sc, a.x_routed, a.x_fp8, a.x_sc,
         a.hidden_fp8, a.hidden_sc) = map(_p, replay)
    _ck(lib.mokb_dispatch_mlp_swiglu_combine_bwd_mxfp8(ctypes.byref(a), _stream()))
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_fp8, d_gate_sc, d_up_shared, d_up_fp8, d_up_sc,
            d_hidden_shared, d_hidden_routed, d_y_fp8, d_y_sc, d_w_shared_gate, d_w_routed_gate, d_w_shared_up,
            d_w_routed_up, d_w_shared_down, d_w_routed_down)
