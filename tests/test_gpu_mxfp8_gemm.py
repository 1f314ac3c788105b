"""GPU parity of the block-scaled MXFP8 grouped GEMM against fp32 matmuls of the de-quantised
operands (products of E4M3 values and power-of-two scales are exact in fp32, so only the
summation order and the final bf16 rounding differ)."""
import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.gpu_common import GEMM_TOL, assert_close

pytestmark = pytest.mark.gpu


def quant(x):
    """bf16 [.., R, C] -> (fp8 cuda, packed scales cuda, de-quantised fp32 cpu), blocks along the last axis."""
    q, s, _, _ = O.mxfp8_quantize(x, True, False)
    deq = O.dequantize(q.reshape(-1, x.shape[-1]), s).reshape(x.shape)
    return q.cuda(), s.cuda(), deq


def groups(rows_per_group):
    offs = np.concatenate([[0], np.cumsum(rows_per_group)]).astype(np.int32)
    gob = np.concatenate([np.full(n // 128, g, np.int32) for g, n in enumerate(rows_per_group)] or [np.zeros(0, np.int32)])
    return torch.from_numpy(offs).cuda(), torch.from_numpy(gob).cuda(), int(offs[-1])


@pytest.mark.parametrize("dual", [False, True])
@pytest.mark.parametrize("rows_per_group,N,K", [([256], 256, 128), ([512, 0, 256], 384, 512), ([256, 768], 256, 1024)])
def test_mxfp8_gemm_nt(rows_per_group, N, K, dual):
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(31)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    W = (torch.randn(G_, N, K, generator=g) * 0.1).to(torch.bfloat16)
    Aq, As, Ad = quant(A)
    Wq, Ws, Wd = quant(W)
    extra = {}
    if dual:
        A2 = torch.randn(rows, K, generator=g).to(torch.bfloat16)
        W2 = (torch.randn(G_, N, K, generator=g) * 0.1).to(torch.bfloat16)
        A2q, A2s, A2d = quant(A2)
        W2q, W2s, W2d = quant(W2)
        extra = dict(A2=A2q, A2_sc=A2s, B2=W2q, B2_sc=W2s)
    D = torch.full((rows, N), 3.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(0, Aq, As, Wq, Ws, D, group_of_block=gob, G=G_, N=N, K=K, **extra)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        ref = Ad[s:e] @ Wd[gi].T
        if dual:
            ref = ref + A2d[s:e] @ W2d[gi].T
        assert_close(f"group {gi}", ref.to(torch.bfloat16), D[s:e], GEMM_TOL)


def test_mxfp8_gemm_dual_b():
    from mok import _C
    rows_per_group, N, K = [512, 256], 384, 256
    offs, gob, rows = groups(rows_per_group)
    g = torch.Generator().manual_seed(32)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    Wg = (torch.randn(2, N, K, generator=g) * 0.1).to(torch.bfloat16)
    Wu = (torch.randn(2, N, K, generator=g) * 0.1).to(torch.bfloat16)
    Aq, As, Ad = quant(A)
    Gq, Gs, Gd = quant(Wg)
    Uq, Us, Ud = quant(Wu)
    D = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    D2 = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(1, Aq, As, Gq, Gs, D, group_of_block=gob, G=2, N=N, K=K, B2=Uq, B2_sc=Us, D2=D2)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(2):
        s, e = int(o[gi]), int(o[gi + 1])
        assert_close("gate", (Ad[s:e] @ Gd[gi].T).to(torch.bfloat16), D[s:e], GEMM_TOL)
        assert_close("up", (Ad[s:e] @ Ud[gi].T).to(torch.bfloat16), D2[s:e], GEMM_TOL)


@pytest.mark.parametrize("limit", [None, 0.5])
def test_mxfp8_gemm_gate_up_swiglu_quant_equals_the_unfused_sequence(limit):
    """Mode 3 (SwiGLU + quantisation in the gate/up epilogue) against mode 1 followed by the quantiser: gate and up
    byte-exact; hidden (computed with the fast division) within one E4M3 step of quantising the bf16 SwiGLU of the
    same gate / up; scale layouts as the quantiser emits them."""
    from mok import _C, ops
    rows_per_group, N, K = [512, 256, 768], 384, 256
    offs, gob, rows = groups(rows_per_group)
    g = torch.Generator().manual_seed(33)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    Wg = (torch.randn(3, N, K, generator=g) * 0.15).to(torch.bfloat16)
    Wu = (torch.randn(3, N, K, generator=g) * 0.15).to(torch.bfloat16)
    Aq, As, _ = quant(A)
    Gq, Gs, _ = quant(Wg)
    Uq, Us, _ = quant(Wu)
    gate = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    up = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(1, Aq, As, Gq, Gs, gate, group_of_block=gob, G=3, N=N, K=K, B2=Uq, B2_sc=Us, D2=up)
    u8 = dict(dtype=torch.uint8, device="cuda")
    outs = [torch.zeros(rows, N, **u8), torch.zeros(rows // 128, N // 128, 32, 16, **u8),
            torch.zeros(rows, N, **u8), torch.zeros(rows // 128, N // 128, 32, 16, **u8),
            torch.zeros(rows, N, **u8), torch.zeros(rows // 128, N // 128, 32, 16, **u8),
            torch.zeros(N, rows, **u8), torch.zeros(N // 128, rows // 128, 32, 16, **u8)]
    _C.grouped_gemm_mxfp8(3, Aq, As, Gq, Gs, None, group_of_block=gob, G=3, N=N, K=K, B2=Uq, B2_sc=Us,
                          quantised_outputs=outs, t_rows=rows, swiglu_limit=limit)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    gq, gs, _, _ = ops.mxfp8_quantize(gate, True, False)
    uq, us, _, _ = ops.mxfp8_quantize(up, True, False)
    assert torch.equal(outs[0], gq.view(torch.uint8)) and torch.equal(outs[1], gs)
    assert torch.equal(outs[2], uq.view(torch.uint8)) and torch.equal(outs[3], us)
    hidden = _C.swiglu_fwd(gate, up, limit)
    hq, hs, hqt, hst = ops.mxfp8_quantize(hidden, True, True)
    f8 = torch.float8_e4m3fn
    for name, got_q, got_s, ref_q, ref_s in (("hidden", outs[4], outs[5], hq, hs), ("hidden^T", outs[6], outs[7], hqt, hst)):
        same = (got_q == ref_q.view(torch.uint8)).float().mean().item()
        assert same > 0.995, (name, same)                                   # a different division rounds a few values differently
        a = O.dequantize(got_q.view(f8).cpu(), got_s.cpu())
        b = O.dequantize(ref_q.cpu(), ref_s.cpu())
        assert_close(name, b, a, (0.05, 2e-3))
        assert (got_s != ref_s).float().mean().item() < 0.01, name


@pytest.mark.parametrize("cols_per_group,M,N", [([256], 128, 256), ([512, 0, 256], 256, 384), ([256, 1024], 384, 512)])
def test_mxfp8_gemm_wgrad(cols_per_group, M, N):
    from mok import _C
    offs, gob, cols = groups(cols_per_group)
    G_ = len(cols_per_group)
    g = torch.Generator().manual_seed(33)
    A = torch.randn(M, cols, generator=g).to(torch.bfloat16)       # token axis contiguous, quantised along it
    B = torch.randn(N, cols, generator=g).to(torch.bfloat16)
    Aq, As, Ad = quant(A)
    Bq, Bs, Bd = quant(B)
    D = torch.full((G_, M, N), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(2, Aq, As, Bq, Bs, D, group_offsets=offs, G=G_, M=M, N=N)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if e == s:
            assert torch.all(D[gi] == 0)
            continue
        ref = (Ad[:, s:e] @ Bd[:, s:e].T).to(torch.bfloat16)
        assert_close(f"wgrad {gi}", ref, D[gi], (GEMM_TOL[0] * 8, GEMM_TOL[1]))


@pytest.mark.parametrize("rows_per_group,H,I,window,push", [([512, 256, 0, 768], 512, 384, 512, False),
                                                            ([2048, 512, 3072], 768, 512, 1024, True)])
def test_mxfp8_fused_forward_equals_the_two_launches_bit_for_bit(rows_per_group, H, I, window, push):
    """Mode 4 (gate|up + SwiGLU + quantisation tiles and the down tiles of the same rows in one persistent launch, tied
    by counters) against mode 3 followed by mode 0; with `push`, the down rows go to a (local) peer buffer instead."""
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(35)
    Aq, As, _ = quant(torch.randn(rows, H, generator=g).to(torch.bfloat16))
    Gq, Gs, _ = quant((torch.randn(G_, I, H, generator=g) * 0.1).to(torch.bfloat16))
    Uq, Us, _ = quant((torch.randn(G_, I, H, generator=g) * 0.1).to(torch.bfloat16))
    Dq, Ds, _ = quant((torch.randn(G_, H, I, generator=g) * 0.1).to(torch.bfloat16))
    u8 = dict(dtype=torch.uint8, device="cuda")

    def outs():
        sc = lambda r, c: torch.zeros(r // 128, c // 128, 32, 16, **u8)
        return [torch.zeros(rows, I, **u8), sc(rows, I), torch.zeros(rows, I, **u8), sc(rows, I),
                torch.zeros(rows, I, **u8), sc(rows, I), torch.zeros(I, rows, **u8), sc(I, rows)]
    ref = outs()
    _C.grouped_gemm_mxfp8(3, Aq, As, Gq, Gs, None, group_of_block=gob, G=G_, N=I, K=H, B2=Uq, B2_sc=Us, quantised_outputs=ref, t_rows=rows)
    y_ref = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(0, ref[4].view(torch.float8_e4m3fn), ref[5], Dq, Ds, y_ref, group_of_block=gob, G=G_, N=H, K=I)
    got = outs()
    blk = torch.zeros(rows // 256, dtype=torch.int32, device="cuda")
    nwin = (rows + window - 1) // window
    done = torch.zeros(nwin, dtype=torch.int32, device="cuda")
    y = torch.full((rows, H), 3.0, dtype=torch.bfloat16, device="cuda")
    extra = {}
    if push:      # identity routing to one local "peer": row r goes to slot perm[r]
        perm = torch.randperm(rows, generator=g).to(torch.int32).cuda()
        home = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
        extra = dict(push_ptrs=[home.data_ptr()], push_rank=torch.zeros(rows, dtype=torch.int32, device="cuda"), push_idx=perm)
    _C.grouped_gemm_mxfp8(4, Aq, As, Gq, Gs, None if push else y, group_of_block=gob, G=G_, N=I, K=H, B2=Uq, B2_sc=Us,
                          quantised_outputs=got, t_rows=rows, B3=Dq, B3_sc=Ds, N2=H, ldd=H, window_rows=window, blk_done=blk,
                          win_done=done, **extra)
    torch.cuda.synchronize()
    assert _C.check_status() == 0, _C.status_detail()
    for a, b in zip(ref, got):
        assert torch.equal(a, b)
    if push:
        assert torch.equal(home[perm.long()], y_ref)
    else:
        assert torch.equal(y, y_ref)
    assert blk.tolist() == [I // 128 * 16] * (rows // 256)
    assert done.tolist() == [min(window, rows - c * window) // 256 * (H // 256) * 16 for c in range(nwin)]
