"""CPU restatement of the MoE-layer hot path of cursor/mixture-of-kittens.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA path: it is
imported by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark, never by the product package.  It is written with numpy (integer /
byte work) and torch CPU tensors (bf16 rounding and fp32 matmuls) and follows
the reference file by file; every function names the reference lines it
restates.

Parity pin: the schedule builder, the MXFP8 quantiser, SwiGLU, the two
epilogues and the BF16 layer (forward + backward) are checked against outputs
of the reference's own pure-PyTorch implementation (tests/utils.py of the
reference, executed on CPU) stored under tests/golden/.  The MXFP8 *layer* has
no reference implementation to pin against (the reference compares its MXFP8
kernels with the BF16 reference under a loose tolerance), so that part of the
oracle is pinned only through the quantiser and through the same loose
tolerance.

Conventions
  R  expert-parallel size, T tokens per rank, K top-k, H hidden, I expert width,
  E_l local experts, C schedule capacity, N padded routed rows on this rank.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

EXPERT_PADDING = 256          # csrc/scheduler.cuh:12 (config::EXPERT_PADDING)
SCHEDULE_THREADS = 1024       # csrc/scheduler.cuh:10 (config::NUM_THREADS)


# ----------------------------------------------------------------------------
# Routing schedule (integer, bit-exact)
# ----------------------------------------------------------------------------
def schedule(topk_all: np.ndarray, num_local_experts: int, schedule_capacity: int, rank: int):
    """Routing schedule of one rank.

    Restates csrc/scheduler.cuh:35-147 (count_kernel, pad_kernel,
    schedule_kernel) and equals tests/utils.py:122-176 of the reference:

      * cnt[e][r]  = routes of source rank r that chose local expert e
      * tokens_per_expert[e] = roundup256(sum_r cnt[e][r]); num_tokens = sum_e
      * the j-th matching route of rank r -- j counted in the order "thread
        (route % 1024) ascending, then route // 1024 ascending", which is how
        a 1024-thread block strides over the route list -- lands at row
        base_e + sum_r' min(cnt[e][r'], j) + #{r' < r : cnt[e][r'] > j}
        (round-robin interleave over source ranks, scheduler.cuh:134-139)
      * peer_rank is -1 on padding rows; peer_token_idx there is unspecified
        by the CUDA reference (scheduler.cuh:158) and is returned as -1 here.

    Raises ValueError when the schedule does not fit (the CUDA reference traps,
    scheduler.cuh:86).
    """
    topk_all = np.ascontiguousarray(topk_all)
    R, T, K = topk_all.shape
    routes = T * K
    first = rank * num_local_experts
    flat = topk_all.reshape(R, routes).astype(np.int64)
    local = flat - first
    valid = (local >= 0) & (local < num_local_experts)

    cnt = np.zeros((num_local_experts, R), dtype=np.int64)
    for r in range(R):
        cnt[:, r] = np.bincount(local[r][valid[r]], minlength=num_local_experts)
    tokens_per_expert = (cnt.sum(1) + EXPERT_PADDING - 1) // EXPERT_PADDING * EXPERT_PADDING
    num_tokens = int(tokens_per_expert.sum())
    if num_tokens > schedule_capacity:
        raise ValueError("schedule_capacity is too small for the schedule")
    base = np.concatenate([[0], np.cumsum(tokens_per_expert)[:-1]])

    peer_rank = np.full(schedule_capacity, -1, dtype=np.int32)
    peer_token_idx = np.full(schedule_capacity, -1, dtype=np.int32)

    # visiting order of a 1024-thread block: thread-major
    padded = (routes + SCHEDULE_THREADS - 1) // SCHEDULE_THREADS * SCHEDULE_THREADS
    order = np.arange(padded).reshape(-1, SCHEDULE_THREADS).T.reshape(-1)
    order = order[order < routes]

    for r in range(R):
        e_in_order = local[r][order]
        ok = valid[r][order]
        e_sel = e_in_order[ok]
        route_sel = order[ok]
        # j = rank of the route among same-expert routes of this source rank
        sort = np.argsort(e_sel, kind="stable")
        e_sorted = e_sel[sort]
        starts = np.concatenate([[0], np.cumsum(np.bincount(e_sorted, minlength=num_local_experts))[:-1]])
        j_sorted = np.arange(e_sorted.size) - starts[e_sorted]
        j = np.empty_like(j_sorted)
        j[sort] = j_sorted
        c = cnt[e_sel]                                   # [n, R]
        dst = base[e_sel] + np.minimum(c, j[:, None]).sum(1) + (c[:, :r] > j[:, None]).sum(1)
        peer_rank[dst] = r
        peer_token_idx[dst] = route_sel.astype(np.int32)

    return (peer_rank, peer_token_idx,
            np.array([num_tokens], dtype=np.int32), tokens_per_expert.astype(np.int32))


def schedule_bruteforce(topk_all: np.ndarray, num_local_experts: int, schedule_capacity: int, rank: int):
    """Pure-Python loop version of `schedule` (small cases only): literally
    walks the routes the way the 1024 threads of scheduler.cuh:78-147 do."""
    R, T, K = topk_all.shape
    routes = T * K
    first = rank * num_local_experts
    flat = topk_all.reshape(R, routes)
    cnt = [[0] * R for _ in range(num_local_experts)]
    for r in range(R):
        for i in range(routes):
            e = int(flat[r, i]) - first
            if 0 <= e < num_local_experts:
                cnt[e][r] += 1
    tpe = [(sum(c) + 255) // 256 * 256 for c in cnt]
    peer_rank = [-1] * schedule_capacity
    peer_tok = [-1] * schedule_capacity
    base = 0
    for e in range(num_local_experts):
        for r in range(R):
            j = 0
            for tid in range(SCHEDULE_THREADS):
                for i in range(tid, routes, SCHEDULE_THREADS):
                    if int(flat[r, i]) - first == e:
                        dst = base
                        for rr in range(R):
                            dst += min(cnt[e][rr], j)
                            dst += 1 if (rr < r and cnt[e][rr] > j) else 0
                        peer_rank[dst] = r
                        peer_tok[dst] = i
                        j += 1
        base += tpe[e]
    return (np.array(peer_rank, np.int32), np.array(peer_tok, np.int32),
            np.array([base], np.int32), np.array(tpe, np.int32))


# ----------------------------------------------------------------------------
# MXFP8 quantiser (byte-exact)
# ----------------------------------------------------------------------------
_INV_448 = np.float32(0.002232142857)      # csrc/mxfp8.cuh:56
_SCALE_FLOOR = np.float32(0.000000000001)  # csrc/mxfp8.cuh:56


def _e8m0_round_up(scale: np.ndarray) -> np.ndarray:
    """cvt.rp.satfinite.ue8m0x2.f32 (csrc/mxfp8.cuh:58): smallest power of two
    >= scale, as a biased exponent byte, saturated to [0, 254]."""
    m, e = np.frexp(scale.astype(np.float32))       # scale = m * 2^e, m in [0.5, 1)
    exp = np.where(m == np.float32(0.5), e - 1, e)  # exact powers of two stay
    return np.clip(exp + 127, 0, 254).astype(np.uint8)


def quantize_blocks(x_bf16: torch.Tensor):
    """Quantise along the last axis in blocks of 32.

    Restates quantize_single_block, csrc/mxfp8.cuh:45-72: amax of the block,
    scale = max(amax * (1/448), 1e-12) rounded UP to a power of two, elements
    multiplied by the exact reciprocal and converted to E4M3 round-to-nearest-
    even, saturating.  An all-zero block therefore gets scale byte 88
    (2^-39 >= 1e-12), where the reference's PyTorch formula
    (tests/utils.py:191-197) would give byte 0; the CUDA behaviour is kept.

    Returns (fp8 bytes as uint8 tensor of x's shape, scale bytes uint8 [..., cols/32]).
    """
    assert x_bf16.dtype == torch.bfloat16 and x_bf16.shape[-1] % 32 == 0
    xf = x_bf16.float().numpy()
    blocks = xf.reshape(*xf.shape[:-1], xf.shape[-1] // 32, 32)
    amax = np.abs(blocks).max(-1).astype(np.float32)
    scale = np.maximum(amax * _INV_448, _SCALE_FLOOR).astype(np.float32)
    byte = _e8m0_round_up(scale)
    inv = np.ldexp(np.float32(1.0), 127 - byte.astype(np.int32)).astype(np.float32)
    scaled = (blocks * inv[..., None]).astype(np.float32).reshape(xf.shape)
    scaled = np.clip(scaled, -448.0, 448.0)
    q = torch.from_numpy(scaled).to(torch.float8_e4m3fn).view(torch.uint8)
    return q, torch.from_numpy(byte)


def pack_scales(scale_bytes: torch.Tensor) -> torch.Tensor:
    """[rows, cols/32] scale bytes -> [rows/128, cols/128, 32, 16]: the byte of
    (row r, 32-column block kb) of a 128x128 tile sits at (r % 32) * 16 +
    (r // 32) * 4 + kb (csrc/mxfp8.cuh:184; tests/utils.py:198-200)."""
    rows, kblocks = scale_bytes.shape
    assert rows % 128 == 0 and kblocks % 4 == 0
    s = scale_bytes.reshape(rows // 128, 4, 32, kblocks // 4, 4)   # [rb, r/32, r%32, cb, kb]
    s = s.permute(0, 3, 2, 1, 4)                                   # [rb, cb, r%32, r/32, kb]
    return s.reshape(rows // 128, kblocks // 4, 32, 16).contiguous()


def unpack_scales(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of `pack_scales`."""
    rb, cb = packed.shape[:2]
    s = packed.reshape(rb, cb, 32, 4, 4).permute(0, 3, 2, 1, 4)
    return s.reshape(rb * 128, cb * 4).contiguous()


def mxfp8_quantize(x_bf16: torch.Tensor, return_normal: bool, return_transposed: bool):
    """quantize_entrypoint, csrc/mxfp8.cuh:234-278 / tests/utils.py:205-221:
    x [M,N] or [E,M,N] -> (x_fp8, x_sc, x_fp8_t, x_sc_t); the transposed pair
    is the quantisation of x^T."""
    def one(x):
        is2d = x.ndim == 2
        x3 = x.unsqueeze(0) if is2d else x
        E, M, N = x3.shape
        q, s = quantize_blocks(x3.reshape(E * M, N).contiguous())
        q = q.reshape(E, M, N).view(torch.float8_e4m3fn)
        return (q.squeeze(0) if is2d else q), pack_scales(s)
    out = [None, None, None, None]
    if return_normal:
        out[0], out[1] = one(x_bf16)
    if return_transposed:
        out[2], out[3] = one(x_bf16.transpose(-2, -1).contiguous())
    return tuple(out)


def dequantize(fp8: torch.Tensor, packed_scales: torch.Tensor) -> torch.Tensor:
    """dequantize_single_block, csrc/mxfp8.cuh:74-90: value * 2^(byte-127), fp32."""
    shape = fp8.shape
    q = fp8.reshape(-1, shape[-1])
    s = unpack_scales(packed_scales).to(torch.int32)
    scale = torch.from_numpy(np.ldexp(np.float32(1.0), (s.numpy() - 127))).float()
    return (q.float().reshape(q.shape[0], -1, 32) * scale[:, :, None]).reshape(shape)


# ----------------------------------------------------------------------------
# SwiGLU
# ----------------------------------------------------------------------------
def swiglu_fwd(gate: torch.Tensor, up: torch.Tensor, limit: float | None) -> torch.Tensor:
    """hidden = bf16(silu(g) * u) from bf16 gate/up in fp32, with the optional
    clamp g <- min(g, L), u <- clamp(u, -L, L)
    (csrc/megakernel/swiglu.cuh:135-147; tests/utils.py:224-235)."""
    g, u = gate.float(), up.float()
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (g / (1.0 + torch.exp(-g)) * u).to(torch.bfloat16)


def swiglu_bwd(gate: torch.Tensor, up: torch.Tensor, d_hidden: torch.Tensor, limit: float | None):
    """swiglu_bwd_pair, csrc/megakernel/swiglu.cuh:1-36.  Inputs fp32-convertible;
    returns (d_gate bf16, d_up bf16, hidden fp32 unrounded)."""
    g, u, dh = gate.float(), up.float(), d_hidden.float()
    if limit is not None:
        gate_ok = g <= limit
        up_ok = (u >= -limit) & (u <= limit)
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    sig = 1.0 / (1.0 + torch.exp(-g))
    silu = g * sig
    dsilu = (1.0 - silu) * sig + silu
    d_gate = dsilu * u * dh
    d_up = silu * dh
    if limit is not None:
        d_gate = torch.where(gate_ok, d_gate, torch.zeros_like(d_gate))
        d_up = torch.where(up_ok, d_up, torch.zeros_like(d_up))
    return d_gate.to(torch.bfloat16), d_up.to(torch.bfloat16), silu * u


# ----------------------------------------------------------------------------
# Epilogues
# ----------------------------------------------------------------------------
def fwd_epilogue(y_shared: torch.Tensor, combine_buffer: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
    """out[t] = bf16(y_shared[t] + sum_k w[t,k] * combine[t*K+k]) accumulated in
    fp32 with k ascending (csrc/utils.cuh:43-95; tests/utils.py:299-307)."""
    T, H = y_shared.shape
    K = topk_weights.shape[1]
    acc = y_shared.float().clone()
    routed = combine_buffer.view(T, K, H)
    for k in range(K):
        acc += routed[:, k].float() * topk_weights[:, k:k + 1]
    return acc.to(torch.bfloat16)


def bwd_epilogue(d_x_shared: torch.Tensor, d_x_routed_buffer: torch.Tensor) -> torch.Tensor:
    """d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed[t*K+k]), fp32, k ascending
    (csrc/utils.cuh:140-176; tests/utils.py:310-317)."""
    T, H = d_x_shared.shape
    K = d_x_routed_buffer.shape[0] // T
    acc = d_x_shared.float().clone()
    routed = d_x_routed_buffer.view(T, K, H)
    for k in range(K):
        acc += routed[:, k].float()
    return acc.to(torch.bfloat16)


# ----------------------------------------------------------------------------
# The layer: forward + backward, all EP ranks simulated in one process
# ----------------------------------------------------------------------------
def _mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """fp32-accumulated product of two tensors given in fp32, rounded to bf16:
    the numerical contract of every grouped GEMM
    (csrc/megakernel/grouped_gemm.cuh:261-294: TMEM fp32 -> bf16 store)."""
    return (a @ b).to(torch.bfloat16)


@dataclass
class RankInputs:
    """One rank's arguments of functional.forward/backward (mok/functional.py:470-500,652-693)."""
    x: torch.Tensor                # [T,H] bf16
    top_experts: torch.Tensor      # [T,K] int64
    router_weights: torch.Tensor   # [T,K] f32
    w_shared_gate: torch.Tensor    # [I,H] bf16
    w_shared_up: torch.Tensor      # [I,H]
    w_shared_down: torch.Tensor    # [H,I]
    w_routed_gate: torch.Tensor    # [E_l,I,H]
    w_routed_up: torch.Tensor      # [E_l,I,H]
    w_routed_down: torch.Tensor    # [E_l,H,I]
    grad_output: torch.Tensor      # [T,H] bf16


class Quantised:
    """MXFP8 operand: dequantised fp32 view of (fp8, packed scales) along the last axis."""
    def __init__(self, x_bf16: torch.Tensor):
        rows = x_bf16.reshape(-1, x_bf16.shape[-1])
        q, s = quantize_blocks(rows.contiguous())
        self.fp8 = q.view(torch.float8_e4m3fn).reshape(x_bf16.shape)
        self.scales = s
        scale = torch.from_numpy(np.ldexp(np.float32(1.0), s.numpy().astype(np.int32) - 127)).float()
        self.deq = (q.view(torch.float8_e4m3fn).float().reshape(rows.shape[0], -1, 32)
                    * scale[:, :, None]).reshape(x_bf16.shape)


def layer_forward_backward(ranks: list[RankInputs], *, schedule_capacity_factor: int = 2,
                           swiglu_limit: float | None = None, mxfp8: bool = False,
                           with_backward: bool = True):
    """Whole layer for all R ranks, following the kernels' dataflow.

    BF16 (mxfp8=False) restates csrc/megakernel/forward.cuh:159-254 and
    backward.cuh:212-418 with the rounding points of the CUDA path: every GEMM
    output, SwiGLU output and scaled d_y row is rounded to bf16
    (grouped_gemm.cuh:261-294, swiglu.cuh:135-168, dispatch_combine.cuh:116-126);
    it agrees with tests/utils.py:320-432 within BF16 tolerance.

    MXFP8 (mxfp8=True): routed GEMM operands are quantised per 32 elements along
    the contraction axis at the points the CUDA path quantises them
    (dispatch_combine.cuh:88-114, grouped_gemm.cuh:295-359, swiglu.cuh:170-185,
    381-441, backward.cuh:335-403); the shared expert stays BF16
    (grouped_gemm.cuh:46).

    Returns a list (one per rank) of dicts with the schedule, the saved forward
    context, `output`, and -- if with_backward -- all gradients.
    """
    R = len(ranks)
    T, H = ranks[0].x.shape
    K = ranks[0].top_experts.shape[1]
    E_l, I, _ = ranks[0].w_routed_gate.shape
    C = T * K * schedule_capacity_factor
    topk_all = np.stack([r.top_experts.numpy().astype(np.int32) for r in ranks])
    lim = swiglu_limit

    def q_or_f(t):          # operand for a routed GEMM, contraction along last axis
        return Quantised(t).deq if mxfp8 else t.float()

    outs = [dict() for _ in range(R)]
    combine = [torch.zeros(T * K, H, dtype=torch.bfloat16) for _ in range(R)]
    d_x_routed_buf = [torch.zeros(T * K, H, dtype=torch.bfloat16) for _ in range(R)]
    d_router_w = [torch.zeros(T * K, dtype=torch.float32) for _ in range(R)]

    for r in range(R):
        inp = ranks[r]
        o = outs[r]
        pr, pt, nt, tpe = schedule(topk_all, E_l, C, r)
        N = int(nt[0])
        o.update(peer_rank=pr, peer_token_idx=pt, num_tokens=nt, tokens_per_expert=tpe)
        pr_t = torch.from_numpy(pr[:N].astype(np.int64))
        pt_t = torch.from_numpy(pt[:N].astype(np.int64))
        real = pr_t >= 0
        # dispatch: pull x rows from the home rank; padding rows are zero (dispatch_combine.cuh:74-83)
        x_routed = torch.zeros(N, H, dtype=torch.bfloat16)
        w_row = torch.zeros(N, dtype=torch.float32)
        for src in range(R):
            m = pr_t == src
            x_routed[m] = ranks[src].x[pt_t[m] // K]
            w_row[m] = ranks[src].router_weights.reshape(-1)[pt_t[m]]
        seg = np.concatenate([[0], np.cumsum(tpe)]).astype(np.int64)

        gate = torch.zeros(N, I, dtype=torch.bfloat16)
        up = torch.zeros_like(gate)
        y = torch.zeros(N, H, dtype=torch.bfloat16)
        for e in range(E_l):
            s, t_ = int(seg[e]), int(seg[e + 1])
            if s == t_:
                continue
            a = q_or_f(x_routed[s:t_])
            gate[s:t_] = _mm(a, q_or_f(inp.w_routed_gate[e]).T)
            up[s:t_] = _mm(a, q_or_f(inp.w_routed_up[e]).T)
        if mxfp8:   # gate/up are saved quantised and SwiGLU reads the bf16 tile (grouped_gemm.cuh:318-338)
            gate_saved, up_saved = Quantised(gate).deq, Quantised(up).deq
        else:
            gate_saved, up_saved = gate.float(), up.float()
        hidden = swiglu_fwd(gate, up, lim)
        for e in range(E_l):
            s, t_ = int(seg[e]), int(seg[e + 1])
            if s == t_:
                continue
            y[s:t_] = _mm(q_or_f(hidden[s:t_]), q_or_f(inp.w_routed_down[e]).T)
        # combine: push rows home (dispatch_combine.cuh:237-238)
        for dst in range(R):
            m = pr_t == dst
            combine[dst][pt_t[m]] = y[m]
        # shared expert (always bf16)
        gate_s = _mm(inp.x.float(), inp.w_shared_gate.float().T)
        up_s = _mm(inp.x.float(), inp.w_shared_up.float().T)
        hidden_s = swiglu_fwd(gate_s, up_s, lim)
        y_s = _mm(hidden_s.float(), inp.w_shared_down.float().T)
        o.update(x_routed=x_routed, gate_routed=gate, up_routed=up, hidden_routed=hidden, y_routed=y,
                 gate_shared=gate_s, up_shared=up_s, hidden_shared=hidden_s, y_shared=y_s,
                 _w_row=w_row, _real=real, _seg=seg, _pr=pr_t, _pt=pt_t,
                 _gate_saved=gate_saved, _up_saved=up_saved)

    for r in range(R):
        outs[r]["combine_buffer"] = combine[r]
        outs[r]["output"] = fwd_epilogue(outs[r]["y_shared"], combine[r], ranks[r].router_weights)
    if not with_backward:
        return outs

    for r in range(R):
        inp, o = ranks[r], outs[r]
        N = int(o["num_tokens"][0])
        pr_t, pt_t, seg, w_row = o["_pr"], o["_pt"], o["_seg"], o["_w_row"]
        # reverse combine: pull d_y rows, scale by the router weight in fp32, round (dispatch_combine.cuh:116-126)
        d_y = torch.zeros(N, H, dtype=torch.bfloat16)
        for src in range(R):
            m = pr_t == src
            d_y[m] = (ranks[src].grad_output[pt_t[m] // K].float() * w_row[m, None]).to(torch.bfloat16)
        d_hidden = torch.zeros(N, I, dtype=torch.bfloat16)
        d_x = torch.zeros(N, H, dtype=torch.bfloat16)
        dWg = torch.zeros(E_l, I, H, dtype=torch.bfloat16)
        dWu = torch.zeros_like(dWg)
        dWd = torch.zeros(E_l, H, I, dtype=torch.bfloat16)
        for e in range(E_l):
            s, t_ = int(seg[e]), int(seg[e + 1])
            if s == t_:
                continue
            # dgrad down: contraction over H; MXFP8 uses W_down^T quantised along H (backward.cuh:335-345)
            wd_t = inp.w_routed_down[e].T.contiguous()          # [I,H]
            d_hidden[s:t_] = _mm(q_or_f(d_y[s:t_]), q_or_f(wd_t).T)
        d_gate, d_up, hidden_f = swiglu_bwd(o["_gate_saved"], o["_up_saved"], d_hidden, lim)
        inv_w = torch.where(w_row > 0, 1.0 / w_row, torch.zeros_like(w_row))
        # router-weight gradient partials (swiglu.cuh:391,444-447)
        d_w_row = (d_hidden.float() * inv_w[:, None] * hidden_f).sum(1)
        for e in range(E_l):
            s, t_ = int(seg[e]), int(seg[e + 1])
            if s == t_:
                continue
            wg_t = inp.w_routed_gate[e].T.contiguous()          # [H,I], contraction over I
            wu_t = inp.w_routed_up[e].T.contiguous()
            acc = q_or_f(d_gate[s:t_]) @ q_or_f(wg_t).T + q_or_f(d_up[s:t_]) @ q_or_f(wu_t).T
            d_x[s:t_] = acc.to(torch.bfloat16)
            # wgrads: contraction over the expert's rows; MXFP8 quantises the transposed
            # activations along the token axis (backward.cuh:369-403)
            def tq(t):
                return q_or_f(t.T.contiguous())
            dWd[e] = _mm(tq(d_y[s:t_]), tq(o["hidden_routed"][s:t_]).T)
            dWg[e] = _mm(tq(d_gate[s:t_]), tq(o["x_routed"][s:t_]).T)
            dWu[e] = _mm(tq(d_up[s:t_]), tq(o["x_routed"][s:t_]).T)
        for dst in range(R):
            m = pr_t == dst
            d_x_routed_buf[dst][pt_t[m]] = d_x[m]
            d_router_w[dst][pt_t[m]] = d_w_row[m]
        # shared expert backward (bf16)
        g = inp.grad_output
        d_hidden_s = _mm(g.float(), inp.w_shared_down.float())
        d_gate_s, d_up_s, _ = swiglu_bwd(o["gate_shared"], o["up_shared"], d_hidden_s, lim)
        d_x_s = (d_gate_s.float() @ inp.w_shared_gate.float()
                 + d_up_s.float() @ inp.w_shared_up.float()).to(torch.bfloat16)
        o.update(d_y_routed=d_y, d_hidden_routed=d_hidden, d_gate_routed=d_gate, d_up_routed=d_up,
                 d_x_routed=d_x, d_w_routed_gate=dWg, d_w_routed_up=dWu, d_w_routed_down=dWd,
                 d_hidden_shared=d_hidden_s, d_gate_shared=d_gate_s, d_up_shared=d_up_s, d_x_shared=d_x_s,
                 d_w_shared_down=_mm(g.float().T, o["hidden_shared"].float()),
                 d_w_shared_gate=_mm(d_gate_s.float().T, inp.x.float()),
                 d_w_shared_up=_mm(d_up_s.float().T, inp.x.float()))
    for r in range(R):
        o = outs[r]
        o["d_x_routed_buffer"] = d_x_routed_buf[r]
        o["d_router_weights"] = d_router_w[r].view(T, K)
        o["d_x"] = bwd_epilogue(o["d_x_shared"], d_x_routed_buf[r])
    return outs


# ----------------------------------------------------------------------------
# Synthetic inputs (the distributions named by the benchmark configurations)
# ----------------------------------------------------------------------------
def make_inputs(*, R: int, T: int, H: int, I: int, E: int, K: int, seed: int = 0,
                routing: str = "gaussian", zipf_s: float = 1.2) -> list[RankInputs]:
    """Seeded CPU inputs: x, grad_out ~ N(0,1) bf16; weights ~ N(0, 0.02^2) bf16;
    routing "router" = top-k of x @ W_r with W_r ~ N(0, 0.02^2), "gaussian" =
    top-k of N(0,1) logits, "zipf" = N(0,1) logits + log-Zipf(s) bias under a
    seeded permutation of experts; router weights = softmax over the selected
    logits (tests/utils.py:82-84 of the reference)."""
    E_l = E // R
    shared = torch.Generator().manual_seed(seed + 7919)
    bias = None
    if routing == "zipf":
        perm = torch.randperm(E, generator=shared)
        bias = torch.empty(E)
        bias[perm] = -zipf_s * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
    w_r = torch.randn(H, E, generator=shared) * 0.02 if routing == "router" else None
    out = []
    for r in range(R):
        g = torch.Generator().manual_seed(seed + r)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        if routing == "router":
            logits = x.float() @ w_r
        else:
            logits = torch.randn(T, E, generator=g)
            if bias is not None:
                logits = logits + bias
        vals, idx = torch.topk(logits, K, dim=1)
        rw = torch.softmax(vals.float(), dim=-1)

        def w(*shape):
            return (torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16)
        out.append(RankInputs(
            x=x, top_experts=idx.to(torch.int64), router_weights=rw,
            w_shared_gate=w(I, H), w_shared_up=w(I, H), w_shared_down=w(H, I),
            w_routed_gate=w(E_l, I, H), w_routed_up=w(E_l, I, H), w_routed_down=w(E_l, H, I),
            grad_output=torch.randn(T, H, generator=g).to(torch.bfloat16)))
    return out


def error_stats(reference: torch.Tensor, actual: torch.Tensor) -> tuple[float, float]:
    """(max |diff|, sum|diff| / sum|ref|): the reference's metric, tests/utils.py:435-457."""
    ref, act = reference.float(), actual.float()
    diff = (ref - act).abs()
    return diff.max().item(), (diff.sum() / ref.abs().sum().clamp_min(1e-30)).item()


BF16_TOLERANCE = (0.5, 0.01)    # tests/utils.py:7
MXFP8_TOLERANCE = (1.0, 0.1)    # tests/utils.py:8
