"""ctypes binding of libmok_b200.so: the module that plays the role of the
reference's pybind11 extension `mok._C` (csrc/bindings.cu:6-94 of the reference).

Each function takes the arguments the reference's `_C` function of the same
name takes (torch tensors, Python ints, pointer lists), allocates the outputs
the reference allocates (with torch.empty, i.e. through the caching allocator:
no cudaMalloc on the step path), and calls the C-ABI entry point on torch's
current stream.  There is no fallback: if the shared library is missing the
import fails, and a failed call raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libmok_b200.so")
if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with `python mixture-of-kittens_b200/build.py` "
        "(the CUDA path has no CPU or PyTorch fallback)")
lib = ctypes.CDLL(_LIB_PATH)

c_int, c_i64, c_f32, c_vp, c_sz = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
c_u64p = ctypes.POINTER(ctypes.c_uint64)

(ST_OK, ST_SCHEDULE_OVERFLOW, ST_BARRIER_TIMEOUT, ST_PIPELINE_TIMEOUT, ST_MACROBATCH_OVERFLOW, ST_FLAG_TIMEOUT,
 ST_BAD_INDEX) = range(7)
STATUS_TEXT = {
    ST_OK: "ok",
    ST_SCHEDULE_OVERFLOW: "the padded routed rows exceed schedule_capacity",
    ST_BARRIER_TIMEOUT: "a rank did not arrive at barrier_all in time",
    ST_PIPELINE_TIMEOUT: "a pipeline wait inside a GEMM kernel ran out",
    ST_MACROBATCH_OVERFLOW: "the padded routed rows exceed macrobatch_size",
    ST_FLAG_TIMEOUT: "a wait on a counter raised by another kernel or CTA ran out",
    ST_BAD_INDEX: "a schedule entry names a route outside [0, tokens * topk); the row was skipped",
}


class FwdArgs(ctypes.Structure):
    _fields_ = (
        [(n, c_int) for n in ("ep_size", "ep_rank", "num_local_tokens", "hidden", "intermediate", "num_local_experts",
                              "topk", "schedule_capacity", "macrobatch_size", "minibatch_size", "num_comm_sms",
                              "has_swiglu_limit")]
        + [("swiglu_limit", c_f32)]
        + [(n, c_vp) for n in ("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert")]
        + [("x_ptrs_host", c_u64p), ("combine_ptrs_host", c_u64p)]
        + [(n, c_vp) for n in ("w_shared_gate", "w_shared_up", "w_shared_down", "w_routed_gate", "w_routed_up",
                               "w_routed_down", "x_routed", "gate_shared", "up_shared", "hidden_shared", "gate_routed",
                               "up_routed", "hidden_routed", "y_shared", "y_routed", "scratch", "status")]
        + [("skip_down_combine", c_int)])


class BwdArgs(ctypes.Structure):
    _fields_ = (
        [(n, c_int) for n in ("ep_size", "ep_rank", "num_local_tokens", "hidden", "intermediate", "num_local_experts",
                              "topk", "schedule_capacity", "macrobatch_size", "minibatch_size", "num_comm_sms",
                              "has_swiglu_limit")]
        + [("swiglu_limit", c_f32)]
        + [(n, c_vp) for n in ("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert")]
        + [(n, c_u64p) for n in ("d_y_ptrs_host", "d_x_routed_ptrs_host", "router_weight_ptrs_host",
                                 "d_router_weight_ptrs_host", "x_ptrs_host")]
        + [(n, c_vp) for n in ("w_shared_gate", "w_shared_up", "w_shared_down", "w_routed_gate", "w_routed_up",
                               "w_routed_down", "x_routed", "gate_shared", "gate_routed", "up_shared", "up_routed",
                               "hidden_shared", "hidden_routed", "d_x_shared", "d_x_routed", "d_gate_shared",
                               "d_gate_routed", "d_up_shared", "d_up_routed", "d_hidden_shared", "d_hidden_routed",
                               "d_y_routed", "d_w_shared_gate", "d_w_routed_gate", "d_w_shared_up", "d_w_routed_up",
                               "d_w_shared_down", "d_w_routed_down", "scratch", "status")])


class GemmArgs(ctypes.Structure):
    _fields_ = [("mode", c_int), ("rows_static", c_int), ("row_begin", c_int), ("row_end", c_int), ("num_rows", c_vp), ("group_of_block", c_vp),
                ("group_offsets", c_vp), ("G", c_int), ("M", c_int), ("N", c_int), ("K", c_int),
                ("A", c_vp), ("B", c_vp), ("A2", c_vp), ("B2", c_vp), ("lda", c_int), ("ldb", c_int),
                ("D", c_vp), ("D2", c_vp), ("D3", c_vp), ("ldd", c_int), ("has_swiglu_limit", c_int),
                ("swiglu_limit", c_f32), ("accumulate", c_int), ("status", c_vp),
                ("B3", c_vp), ("D4", c_vp), ("N2", c_int), ("ldb3", c_int), ("ldd4", c_int), ("window_rows", c_int),
                ("win_ready", c_vp), ("win_ready_target", c_int), ("blk_done", c_vp), ("win_done", c_vp),
                ("push_ptrs_host", c_u64p), ("push_ep_size", c_int), ("push_rank", c_vp), ("push_idx", c_vp),
                ("push_values", c_vp), ("push_value_ptrs_host", c_u64p), ("push_index_limit", c_i64), ("group_k_end", c_vp)]


class GemmFp8Args(ctypes.Structure):
    _fields_ = (
        [("mode", c_int), ("rows_static", c_int), ("row_begin", c_int), ("row_end", c_int), ("num_rows", c_vp),
         ("group_of_block", c_vp), ("group_offsets", c_vp), ("G", c_int), ("M", c_int), ("N", c_int), ("K", c_int),
         ("A", c_vp), ("A_sc", c_vp), ("B", c_vp), ("B_sc", c_vp), ("A2", c_vp), ("A2_sc", c_vp), ("B2", c_vp),
         ("B2_sc", c_vp), ("D", c_vp), ("D2", c_vp), ("ldd", c_int), ("t_first", c_int), ("accumulate", c_int)]
        + [(n, c_vp) for n in ("gate_q", "gate_sc", "up_q", "up_sc", "hid_q", "hid_sc", "hid_qt", "hid_sct")]
        + [("t_rows", c_int), ("has_swiglu_limit", c_int), ("swiglu_limit", c_f32), ("status", c_vp)]
        + [("B3", c_vp), ("B3_sc", c_vp), ("N2", c_int), ("window_rows", c_int), ("win_ready", c_vp), ("win_ready_target", c_int),
           ("blk_done", c_vp), ("win_done", c_vp), ("push_ptrs_host", c_u64p), ("push_ep_size", c_int), ("push_rank", c_vp),
           ("push_idx", c_vp), ("push_values", c_vp), ("push_value_ptrs_host", c_u64p), ("push_index_limit", c_i64),
           ("reserve_sms", c_int)])


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_last_error = _sig("mokb_last_error", ctypes.c_char_p)
_sig("mokb_device_arch", c_int)
_sig("mokb_sm_count", c_int)
_sig("mokb_struct_sizes", c_int, ctypes.POINTER(c_int), c_int)
_sig("mokb_set_barrier_timeout_ms", c_int, c_int)
_sig("mokb_launch_count", ctypes.c_ulonglong)
_sig("mokb_trace_begin", c_int, c_vp)
_sig("mokb_trace_end", ctypes.c_longlong, ctypes.c_char_p, c_sz)
_sig("mokb_all_gather_top_experts", c_int, c_vp, c_u64p, c_int, c_int, c_i64, c_vp)
_sig("mokb_barrier_all", c_int, c_u64p, c_int, c_int, c_vp, c_vp, c_vp)
_sig("mokb_schedule_scratch_bytes", c_sz, c_int, c_int)
_sig("mokb_schedule", c_int, c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp)
_sig("mokb_schedule_noalloc", c_int, c_vp, c_int, c_int, c_int, c_int, c_int, c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp)
_sig("mokb_mxfp8_quantize", c_int, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp, c_vp)
_sig("mokb_fwd_epilogue", c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_vp)
_sig("mokb_bwd_epilogue", c_int, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_vp)
_sig("mokb_layer_scratch_bytes", c_sz, c_int, c_int, c_int)
_sig("mokb_dispatch_mlp_swiglu_combine_fwd_bf16", c_int, ctypes.POINTER(FwdArgs), c_vp)
_sig("mokb_dispatch_mlp_swiglu_combine_bwd_bf16", c_int, ctypes.POINTER(BwdArgs), c_vp)
_sig("mokb_grouped_gemm_bf16", c_int, ctypes.POINTER(GemmArgs), c_vp)
_sig("mokb_grouped_gemm_mxfp8", c_int, ctypes.POINTER(GemmFp8Args), c_vp)
_sig("mokb_dispatch_rows", c_int, c_u64p, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_i64, c_vp, c_u64p, c_vp, c_vp)
_sig("mokb_combine_rows", c_int, c_vp, c_u64p, c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_vp, c_u64p, c_vp)
_sig("mokb_comm_default_blocks", c_int)
_sig("mokb_dispatch_rows_window", c_int, c_u64p, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_int, c_i64, c_vp, c_u64p, c_vp, c_int,
     c_vp, c_vp, c_vp, c_i64, c_vp, c_vp)
_sig("mokb_combine_rows_window", c_int, c_vp, c_u64p, c_int, c_vp, c_vp, c_vp, c_int, c_int, c_int, c_i64, c_vp, c_u64p, c_int, c_vp,
     c_int, c_vp, c_i64, c_vp)
_sig("mokb_swiglu_fwd", c_int, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_f32, c_vp)
_sig("mokb_swiglu_bwd", c_int, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_int, c_f32, c_vp)

EXPORTED = [
    "mokb_last_error", "mokb_device_arch", "mokb_sm_count", "mokb_struct_sizes", "mokb_set_barrier_timeout_ms", "mokb_launch_count",
    "mokb_trace_begin", "mokb_trace_end",
    "mokb_all_gather_top_experts", "mokb_barrier_all", "mokb_schedule_scratch_bytes", "mokb_schedule", "mokb_schedule_noalloc",
    "mokb_mxfp8_quantize", "mokb_fwd_epilogue", "mokb_bwd_epilogue", "mokb_layer_scratch_bytes",
    "mokb_dispatch_mlp_swiglu_combine_fwd_bf16", "mokb_dispatch_mlp_swiglu_combine_bwd_bf16",
    "mokb_grouped_gemm_bf16", "mokb_grouped_gemm_mxfp8", "mokb_dispatch_rows", "mokb_combine_rows", "mokb_swiglu_fwd", "mokb_swiglu_bwd",
    "mokb_comm_default_blocks", "mokb_dispatch_rows_window", "mokb_combine_rows_window",
]


def trace_begin():
    """Start recording the launch timeline of this library (diagnostic)."""
    _ck(lib.mokb_trace_begin(_stream()))


def trace_end():
    """Stop recording; returns [(tag, arg, stream_no, begin_ms, end_ms)] for every launcher call since trace_begin."""
    cap = 1 << 20
    buf = ctypes.create_string_buffer(cap)
    need = lib.mokb_trace_end(buf, cap)
    if need < 0:
        raise MokError("trace_end: CUDA error")
    out = []
    for line in buf.value.decode().splitlines():
        tag, arg, sid, t0, t1 = line.split()
        out.append((tag, int(arg), int(sid), float(t0), float(t1)))
    return out


def _check_struct_layout():
    sizes = (c_int * 3)()
    lib.mokb_struct_sizes(sizes, 3)
    mine = (ctypes.sizeof(FwdArgs), ctypes.sizeof(BwdArgs), ctypes.sizeof(GemmArgs))
    if tuple(sizes) != mine:
        raise ImportError(f"struct layout mismatch between _C.py {mine} and libmok_b200.so {tuple(sizes)}")


_check_struct_layout()


class MokError(RuntimeError):
    pass


# The BF16 layer sends the rows of y_routed / d_x_routed to their home ranks from the epilogue of the GEMM that computes
# them, so those two outputs (staging buffers in the reference, read by nothing afterwards) stay unwritten unless this
# is set: MOKB_KEEP_STAGING_ROWS=1 in the environment, or the attribute at run time.
KEEP_STAGING_ROWS = os.environ.get("MOKB_KEEP_STAGING_ROWS", "0") == "1"


def _ck(rc: int) -> None:
    if rc != 0:
        raise MokError(f"mok_b200 error {rc}: {_last_error().decode(errors='replace')}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the raw getter when this torch has it: building a Stream object costs several
    microseconds, and every launcher call asks)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _ptr_array(ptrs: list[int]):
    return (ctypes.c_uint64 * len(ptrs))(*ptrs)


_STATUS: dict[int, torch.Tensor] = {}


def status_tensor(device: torch.device | None = None) -> torch.Tensor:
    """The per-device status word kernels write a code into when something goes wrong."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))      # code + three words of detail
        _STATUS[idx] = t
    return t


def check_status(device: torch.device | None = None, *, reset: bool = True) -> int:
    """Reads the status word (synchronises the host: for tests and debugging, never called by the layer)."""
    t = status_tensor(device)
    words = t.tolist()
    code = int(words[0])
    _LAST_DETAIL[:] = words
    if reset and code:
        t.zero_()
    return code


_LAST_DETAIL = [0, 0, 0, 0]


def status_detail() -> list[int]:
    """The four status words as the last check_status() read them: [code, kind, index, value seen << 16 | target]."""
    return list(_LAST_DETAIL)


def raise_for_status(device: torch.device | None = None) -> None:
    code = check_status(device)
    if code:
        raise MokError(f"device status {code}: {STATUS_TEXT.get(code, 'unknown')}")


_SCRATCH: dict[tuple[int, int], torch.Tensor] = {}


def _layer_scratch(dev: torch.device, nbytes: int) -> torch.Tensor:
    """The layer's work area (tables, counters, per-row router weights): one tensor per (device, stream), grown when a
    call needs more and otherwise reused -- every call's prologue re-initialises what it reads, and calls on one
    stream run one after the other (the reference allocates and zeroes its counters per call, csrc/megakernel/
    forward.cuh:345-368, and marks that as removable)."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream())
    t = _SCRATCH.get(key)
    if t is None or t.numel() < nbytes:
        t = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _SCRATCH[key] = t
    return t


def launch_count() -> int:
    return int(lib.mokb_launch_count())


def set_barrier_timeout_ms(ms: int) -> None:
    _ck(lib.mokb_set_barrier_timeout_ms(int(ms)))


# ----------------------------------------------------------------------------
# The 14 functions of the reference's `_C` (BF16 ones here; MXFP8 in _C_mxfp8)
# ----------------------------------------------------------------------------
def all_gather_top_experts(top_experts, all_gather_top_experts_buffer, multicast_ptr, rank, chunk_bytes, peer_ptrs=None):
    """`multicast_ptr` and `chunk_bytes` are accepted for signature compatibility; the gather uses
    plain stores to each peer's buffer, so the caller passes the peers' unicast addresses."""
    if peer_ptrs is None:
        raise MokError("all_gather_top_experts needs the peers' buffer addresses (peer_ptrs)")
    ep_size = all_gather_top_experts_buffer.shape[0]
    _ck(lib.mokb_all_gather_top_experts(_p(top_experts), _ptr_array(peer_ptrs), ep_size, rank,
                                        top_experts.numel(), _stream()))


def barrier_all(barrier_buffer, barrier_buffer_ptrs, multicast_ptr, target, rank=None):
    ep_size = len(barrier_buffer_ptrs)
    if rank is None:
        rank = barrier_buffer_ptrs.index(barrier_buffer.data_ptr())
    _ck(lib.mokb_barrier_all(_ptr_array(barrier_buffer_ptrs), ep_size, rank, _p(target),
                             _p(status_tensor(barrier_buffer.device)), _stream()))


def schedule(topk_all, num_local_experts, schedule_capacity, rank):
    ep_size, T, K = topk_all.shape
    dev = topk_all.device
    peer_rank = torch.empty(schedule_capacity, dtype=torch.int32, device=dev)
    peer_token_idx = torch.empty(schedule_capacity, dtype=torch.int32, device=dev)
    num_tokens = torch.empty(1, dtype=torch.int32, device=dev)
    tokens_per_expert = torch.empty(num_local_experts, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.mokb_schedule_scratch_bytes(ep_size, num_local_experts), dtype=torch.uint8, device=dev)
    _ck(lib.mokb_schedule(_p(topk_all), ep_size, T, K, num_local_experts, schedule_capacity, rank,
                          _p(peer_rank), _p(peer_token_idx), _p(num_tokens), _p(tokens_per_expert),
                          _p(scratch), _p(status_tensor(dev)), _stream()))
    return peer_rank, peer_token_idx, num_tokens, tokens_per_expert


def schedule_noalloc(topk_all, num_local_experts, schedule_capacity, rank, peer_rank, peer_token_idx, num_tokens,
                     tokens_per_expert):
    """The schedule through the entry point that allocates nothing: the caller hands in all four outputs,
    and the work area is the library's built-in array (limit: 1024 experts over all ranks)."""
    ep_size, T, K = topk_all.shape
    _ck(lib.mokb_schedule_noalloc(_p(topk_all), ep_size, T, K, num_local_experts, schedule_capacity, rank,
                                  _p(peer_rank), _p(peer_token_idx), _p(num_tokens), _p(tokens_per_expert),
                                  _p(status_tensor(topk_all.device)), _stream()))


def mxfp8_quantize(x_bf16, return_normal, return_transposed):
    dev = x_bf16.device
    if x_bf16.ndim == 2:
        E, (M, N) = 1, x_bf16.shape
        lead = ()
    else:
        E, M, N = x_bf16.shape
        lead = (E,)
    q = s = qt = st = None
    if return_normal:
        q = torch.empty(*lead, M, N, dtype=torch.float8_e4m3fn, device=dev)
        s = torch.empty(E * M // 128, N // 128, 32, 16, dtype=torch.uint8, device=dev)
    if return_transposed:
        qt = torch.empty(*lead, N, M, dtype=torch.float8_e4m3fn, device=dev)
        st = torch.empty(E * N // 128, M // 128, 32, 16, dtype=torch.uint8, device=dev)
    _ck(lib.mokb_mxfp8_quantize(_p(x_bf16.contiguous()), E, M, N, _p(q), _p(s), _p(qt), _p(st), _stream()))
    return q, s, qt, st


def fwd_epilogue(y_shared, combine_buffer, topk_weights):
    out = torch.empty_like(y_shared)
    T, H = y_shared.shape
    _ck(lib.mokb_fwd_epilogue(_p(y_shared), _p(combine_buffer), _p(topk_weights), _p(out), T, H,
                              topk_weights.shape[1], _stream()))
    return out


def bwd_epilogue(d_x_shared, d_x_routed_buffer):
    out = torch.empty_like(d_x_shared)
    T, H = d_x_shared.shape
    _ck(lib.mokb_bwd_epilogue(_p(d_x_shared), _p(d_x_routed_buffer), _p(out), T, H,
                              d_x_routed_buffer.shape[0] // T, _stream()))
    return out


def _common(args, *, x_ptrs, x_like, w_shared_gate, w_routed_gate, schedule_peer_rank, schedule_peer_token_idx,
            num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
    T, H = x_like.shape
    I = w_shared_gate.shape[0]
    E_l = w_routed_gate.shape[0]
    ep_size = len(x_ptrs)
    try:
        ep_rank = x_ptrs.index(x_like.data_ptr())
    except ValueError:
        raise MokError("the local buffer's address is not in its peer pointer list") from None
    args.ep_size, args.ep_rank = ep_size, ep_rank
    args.num_local_tokens, args.hidden, args.intermediate, args.num_local_experts, args.topk = T, H, I, E_l, topk
    args.schedule_capacity = schedule_peer_rank.numel()
    args.macrobatch_size, args.minibatch_size, args.num_comm_sms = macrobatch_size, minibatch_size, num_comm_sms
    args.has_swiglu_limit = 0 if swiglu_limit is None else 1
    args.swiglu_limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    args.peer_rank, args.peer_token_idx = _p(schedule_peer_rank), _p(schedule_peer_token_idx)
    args.num_tokens, args.tokens_per_expert = _p(num_tokens), _p(tokens_per_expert)
    dev = x_like.device
    scratch = _layer_scratch(dev, lib.mokb_layer_scratch_bytes(args.schedule_capacity, E_l, macrobatch_size))
    args.scratch = _p(scratch)
    args.status = _p(status_tensor(dev))
    return T, H, I, E_l, dev, scratch


def _fwd_bf16(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
              w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
              topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, skip_down_combine):
    a = FwdArgs()
    T, H, I, E_l, dev, scratch = _common(
        a, x_ptrs=x_ptrs, x_like=x, w_shared_gate=w_shared_gate, w_routed_gate=w_routed_gate,
        schedule_peer_rank=schedule_peer_rank, schedule_peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
        tokens_per_expert=tokens_per_expert, topk=topk, swiglu_limit=swiglu_limit, num_comm_sms=num_comm_sms,
        macrobatch_size=macrobatch_size, minibatch_size=minibatch_size)
    MB = macrobatch_size
    bf = dict(dtype=torch.bfloat16, device=dev)
    x_routed = torch.empty(MB, H, **bf)
    gate_shared, up_shared, hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    gate_routed, up_routed, hidden_routed = (torch.empty(MB, I, **bf) for _ in range(3))
    y_shared = y_routed = None
    keep = [_ptr_array(x_ptrs)]
    a.x_ptrs_host = keep[0]
    if not skip_down_combine:
        y_shared = torch.empty(T, H, **bf)
        y_routed = torch.empty(MB, H, **bf)
        keep.append(_ptr_array(combine_buffer_ptrs))
        a.combine_ptrs_host = keep[1]
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = _p(w_shared_gate), _p(w_shared_up), _p(w_shared_down)
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = _p(w_routed_gate), _p(w_routed_up), _p(w_routed_down)
    a.x_routed = _p(x_routed)
    a.gate_shared, a.up_shared, a.hidden_shared = _p(gate_shared), _p(up_shared), _p(hidden_shared)
    a.gate_routed, a.up_routed, a.hidden_routed = _p(gate_routed), _p(up_routed), _p(hidden_routed)
    # y_routed is the reference's staging buffer of the combine (its rows go to the peers from there); here the rows
    # go to the peers from the GEMM's epilogue and the tensor is only filled on request
    a.y_shared, a.y_routed = _p(y_shared), (_p(y_routed) if KEEP_STAGING_ROWS else None)
    a.skip_down_combine = 1 if skip_down_combine else 0
    _ck(lib.mokb_dispatch_mlp_swiglu_combine_fwd_bf16(ctypes.byref(a), _stream()))
    return x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed, y_shared, y_routed


def dispatch_mlp_swiglu_combine_fwd_bf16(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate,
                                         w_shared_up, w_routed_up, w_shared_down, w_routed_down, schedule_peer_rank,
                                         schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                                         num_comm_sms, macrobatch_size, minibatch_size):
    return _fwd_bf16(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up,
                     w_routed_up, w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx,
                     num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
                     minibatch_size, False)


def recompute_forward_context_bf16(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
                                   schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk,
                                   swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
    return _fwd_bf16(x, x_ptrs, None, None, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, None, None,
                     schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit,
                     num_comm_sms, macrobatch_size, minibatch_size, True)[:7]


def dispatch_mlp_swiglu_combine_bwd_bf16(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs,
                                         router_weight_buffer, router_weight_buffer_ptrs, d_router_weight_buffer,
                                         d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up,
                                         w_routed_up, w_shared_down, w_routed_down, x_routed, gate_shared, gate_routed,
                                         up_shared, up_routed, hidden_shared, hidden_routed, x, x_ptrs,
                                         schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
                                         topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size):
    a = BwdArgs()
    T, H, I, E_l, dev, scratch = _common(
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
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = _p(w_routed_gate), _p(w_routed_up), _p(w_routed_down)
    a.x_routed = _p(x_routed)
    a.gate_shared, a.gate_routed, a.up_shared, a.up_routed = _p(gate_shared), _p(gate_routed), _p(up_shared), _p(up_routed)
    a.hidden_shared, a.hidden_routed = _p(hidden_shared), _p(hidden_routed)
    d_x_shared = torch.empty(T, H, **bf)
    d_x_routed = torch.empty(MB, H, **bf)
    d_gate_shared, d_up_shared, d_hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    d_gate_routed, d_up_routed, d_hidden_routed = (torch.empty(MB, I, **bf) for _ in range(3))
    d_y_routed = torch.empty(MB, H, **bf)
    d_w_shared_gate, d_w_shared_up = torch.empty(I, H, **bf), torch.empty(I, H, **bf)
    d_w_shared_down = torch.empty(H, I, **bf)
    d_w_routed_gate, d_w_routed_up = torch.empty(E_l, I, H, **bf), torch.empty(E_l, I, H, **bf)
    d_w_routed_down = torch.empty(E_l, H, I, **bf)
    a.d_x_shared, a.d_x_routed = _p(d_x_shared), (_p(d_x_routed) if KEEP_STAGING_ROWS else None)
    a.d_gate_shared, a.d_gate_routed, a.d_up_shared, a.d_up_routed = (_p(d_gate_shared), _p(d_gate_routed),
                                                                     _p(d_up_shared), _p(d_up_routed))
    a.d_hidden_shared, a.d_hidden_routed, a.d_y_routed = _p(d_hidden_shared), _p(d_hidden_routed), _p(d_y_routed)
    a.d_w_shared_gate, a.d_w_routed_gate, a.d_w_shared_up, a.d_w_routed_up = (_p(d_w_shared_gate), _p(d_w_routed_gate),
                                                                             _p(d_w_shared_up), _p(d_w_routed_up))
    a.d_w_shared_down, a.d_w_routed_down = _p(d_w_shared_down), _p(d_w_routed_down)
    _ck(lib.mokb_dispatch_mlp_swiglu_combine_bwd_bf16(ctypes.byref(a), _stream()))
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_routed, d_up_shared, d_up_routed, d_hidden_shared,
            d_hidden_routed, d_y_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up,
            d_w_shared_down, d_w_routed_down)


# ----------------------------------------------------------------------------
# Building blocks (tests, micro-benchmarks)
# ----------------------------------------------------------------------------
def grouped_gemm(mode, A, B, D, *, rows=None, num_rows=None, group_of_block=None, group_offsets=None, G=1,
                 M=0, N=0, K=0, A2=None, B2=None, D2=None, D3=None, lda=None, ldb=None, ldd=None, swiglu_limit=None,
                 row_begin=0, row_end=0, accumulate=False, B3=None, D4=None, N2=0, window_rows=0, win_ready=None,
                 win_ready_target=0, blk_done=None, win_done=None, push_ptrs=None, push_rank=None, push_idx=None,
                 push_values=None, push_value_ptrs=None, N2_ld=None, group_k_end=None, push_index_limit=0):
    """Modes 0-3 as in the header; mode 4 = gate/up + SwiGLU (B, B2 -> D, D2, D3) and the down projection
    (D3, B3 -> D4 [rows, N2]) in one launch, with the optional window counters."""
    g = GemmArgs()
    g.B3, g.D4, g.N2 = _p(B3), _p(D4), N2
    g.ldb3 = B3.shape[-1] if B3 is not None else 0
    g.ldd4 = D4.shape[-1] if D4 is not None else (N2_ld or N2)
    keep = []
    if push_ptrs is not None:
        keep.append(_ptr_array(push_ptrs))
        g.push_ptrs_host, g.push_ep_size = keep[-1], len(push_ptrs)
        g.push_rank, g.push_idx, g.push_values = _p(push_rank), _p(push_idx), _p(push_values)
        g.push_index_limit = push_index_limit
        if push_value_ptrs is not None:
            keep.append(_ptr_array(push_value_ptrs))
            g.push_value_ptrs_host = keep[-1]
    g.window_rows, g.win_ready, g.win_ready_target = window_rows, _p(win_ready), win_ready_target
    g.blk_done, g.win_done = _p(blk_done), _p(win_done)
    g.group_k_end = _p(group_k_end)
    g.mode = mode
    g.accumulate = 1 if accumulate else 0
    g.row_begin, g.row_end = row_begin, row_end
    g.rows_static = A.shape[0] if rows is None else rows
    g.num_rows, g.group_of_block, g.group_offsets = _p(num_rows), _p(group_of_block), _p(group_offsets)
    g.G, g.M, g.N, g.K = G, M, N, K
    g.A, g.B, g.A2, g.B2 = _p(A), _p(B), _p(A2), _p(B2)
    g.lda = A.shape[-1] if lda is None else lda
    g.ldb = B.shape[-1] if ldb is None else ldb
    g.D, g.D2, g.D3 = _p(D), _p(D2), _p(D3)
    g.ldd = (D.shape[-1] if D is not None else N) if ldd is None else ldd
    g.has_swiglu_limit = 0 if swiglu_limit is None else 1
    g.swiglu_limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    g.status = _p(status_tensor(A.device))
    _ck(lib.mokb_grouped_gemm_bf16(ctypes.byref(g), _stream()))


def grouped_gemm_mxfp8(mode, A, A_sc, B, B_sc, D, *, rows=None, num_rows=None, group_of_block=None, group_offsets=None,
                       G=1, M=0, N=0, K=0, A2=None, A2_sc=None, B2=None, B2_sc=None, D2=None, ldd=None, row_begin=0, row_end=0,
                       t_first=0, accumulate=False, quantised_outputs=None, t_rows=0, swiglu_limit=None, B3=None, B3_sc=None,
                       N2=0, window_rows=0, win_ready=None, win_ready_target=0, blk_done=None, win_done=None, push_ptrs=None,
                       push_rank=None, push_idx=None, push_values=None, push_value_ptrs=None, reserve_sms=0,
                       push_index_limit=0):
    """`quantised_outputs` (modes 3, 4): (gate_q, gate_sc, up_q, up_sc, hid_q, hid_sc, hid_qt, hid_sct); D is unused in
    mode 3 and the down projection's output [rows, N2] in mode 4 (B3, B3_sc: its weights)."""
    g = GemmFp8Args()
    g.B3, g.B3_sc, g.N2 = _p(B3), _p(B3_sc), N2
    g.reserve_sms = reserve_sms
    g.window_rows, g.win_ready, g.win_ready_target = window_rows, _p(win_ready), win_ready_target
    g.blk_done, g.win_done = _p(blk_done), _p(win_done)
    keep = []
    if push_ptrs is not None:
        keep.append(_ptr_array(push_ptrs))
        g.push_ptrs_host, g.push_ep_size = keep[-1], len(push_ptrs)
        g.push_rank, g.push_idx, g.push_values = _p(push_rank), _p(push_idx), _p(push_values)
        g.push_index_limit = push_index_limit
        if push_value_ptrs is not None:
            keep.append(_ptr_array(push_value_ptrs))
            g.push_value_ptrs_host = keep[-1]
    g.mode = mode
    g.rows_static = (A.shape[0] if mode != 2 else A.shape[1]) if rows is None else rows
    g.row_begin, g.row_end = row_begin, row_end
    g.num_rows, g.group_of_block, g.group_offsets = _p(num_rows), _p(group_of_block), _p(group_offsets)
    g.G, g.M, g.N, g.K = G, M, N, K
    g.A, g.A_sc, g.B, g.B_sc = _p(A), _p(A_sc), _p(B), _p(B_sc)
    g.A2, g.A2_sc, g.B2, g.B2_sc = _p(A2), _p(A2_sc), _p(B2), _p(B2_sc)
    g.D, g.D2 = _p(D), _p(D2)
    g.ldd = (D.shape[-1] if D is not None else N) if ldd is None else ldd
    g.t_first, g.accumulate = t_first, int(bool(accumulate))
    if quantised_outputs is not None:
        (g.gate_q, g.gate_sc, g.up_q, g.up_sc, g.hid_q, g.hid_sc, g.hid_qt, g.hid_sct) = map(_p, quantised_outputs)
        g.t_rows = t_rows
        g.has_swiglu_limit = 0 if swiglu_limit is None else 1
        g.swiglu_limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    g.status = _p(status_tensor(A.device))
    _ck(lib.mokb_grouped_gemm_mxfp8(ctypes.byref(g), _stream()))


def dispatch_rows(src_ptrs, peer_rank, peer_token_idx, num_rows, max_rows, row_divisor, hidden, dst,
                  row_scale_ptrs=None, row_scale_out=None):
    _ck(lib.mokb_dispatch_rows(_ptr_array(src_ptrs), len(src_ptrs), _p(peer_rank), _p(peer_token_idx), _p(num_rows),
                               max_rows, row_divisor, hidden, _p(dst),
                               None if row_scale_ptrs is None else _ptr_array(row_scale_ptrs), _p(row_scale_out),
                               _stream()))


def combine_rows(src, dst_ptrs, peer_rank, peer_token_idx, num_rows, max_rows, hidden, row_values=None, value_ptrs=None):
    _ck(lib.mokb_combine_rows(_p(src), _ptr_array(dst_ptrs), len(dst_ptrs), _p(peer_rank), _p(peer_token_idx),
                              _p(num_rows), max_rows, hidden, _p(row_values),
                              None if value_ptrs is None else _ptr_array(value_ptrs), _stream()))


def comm_default_blocks() -> int:
    return int(lib.mokb_comm_default_blocks())


def dispatch_rows_window(src_ptrs, peer_rank, peer_token_idx, num_rows, max_rows, row_begin, row_end, row_divisor, hidden, dst,
                         row_scale_ptrs=None, row_scale_out=None, blocks=0, done_counter=None, q_out=None, q_sc_out=None,
                         index_limit=0):
    _ck(lib.mokb_dispatch_rows_window(_ptr_array(src_ptrs), len(src_ptrs), _p(peer_rank), _p(peer_token_idx), _p(num_rows),
                                      max_rows, row_begin, row_end, row_divisor, hidden, _p(dst),
                                      None if row_scale_ptrs is None else _ptr_array(row_scale_ptrs), _p(row_scale_out),
                                      blocks, _p(done_counter), _p(q_out), _p(q_sc_out), index_limit,
                                      _p(status_tensor(dst.device)), _stream()))


def combine_rows_window(src, dst_ptrs, peer_rank, peer_token_idx, num_rows, max_rows, row_begin, row_end, hidden,
                        row_values=None, value_ptrs=None, blocks=0, wait_counter=None, arrivals_per_row_block=0,
                        index_limit=0):
    _ck(lib.mokb_combine_rows_window(_p(src), _ptr_array(dst_ptrs), len(dst_ptrs), _p(peer_rank), _p(peer_token_idx),
                                     _p(num_rows), max_rows, row_begin, row_end, hidden, _p(row_values),
                                     None if value_ptrs is None else _ptr_array(value_ptrs), blocks, _p(wait_counter),
                                     arrivals_per_row_block, _p(status_tensor(src.device)), index_limit, _stream()))


def swiglu_fwd(gate, up, swiglu_limit=None, num_rows=None):
    hidden = torch.empty_like(gate)
    _ck(lib.mokb_swiglu_fwd(_p(gate), _p(up), _p(hidden), _p(num_rows), gate.shape[0], gate.shape[1],
                            0 if swiglu_limit is None else 1, 0.0 if swiglu_limit is None else float(swiglu_limit),
                            _stream()))
    return hidden


def swiglu_bwd(gate, up, d_hidden, swiglu_limit=None, row_scale=None, want_row_grad=False, num_rows=None):
    d_gate, d_up = torch.empty_like(gate), torch.empty_like(up)
    row_grad = torch.empty(gate.shape[0], dtype=torch.float32, device=gate.device) if want_row_grad else None
    _ck(lib.mokb_swiglu_bwd(_p(gate), _p(up), _p(d_hidden), _p(d_gate), _p(d_up), _p(row_scale), _p(row_grad),
                            _p(num_rows), gate.shape[0], gate.shape[1], 0 if swiglu_limit is None else 1,
                            0.0 if swiglu_limit is None else float(swiglu_limit), _stream()))
    return d_gate, d_up, row_grad
