"""GPU parity tests of the individual kernels, through the C-ABI (mok._C / mok.ops),
against the CPU oracle and the golden fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.golden import make_golden as G
from tests.gpu_common import GEMM_TOL, assert_close

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def mods():
    from mok import _C, ops
    return _C, ops


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(HERE, "golden", "ops_golden.npz"))


def bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


# ------------------------------------------------------------------ schedule
def run_schedule(ops, _C, topk, E_l, C, rank):
    out = ops.schedule(torch.from_numpy(topk).cuda(), E_l, C, rank)
    code = _C.check_status()
    return [o.cpu().numpy() for o in out], code


@pytest.mark.parametrize("case", G.SCHEDULE_CASES, ids=lambda c: c[0])
def test_schedule_bit_exact_vs_golden(mods, golden, case):
    _C, ops = mods
    name, R, T, K, E_l, factor, pattern = case
    topk = G.schedule_topk(R, T, K, E_l, pattern)
    for rank in sorted({0, R - 1}):
        (pr, pt, nt, tpe), code = run_schedule(ops, _C, topk, E_l, T * K * factor, rank)
        assert code == 0
        key = f"sched_{name}_rank{rank}"
        np.testing.assert_array_equal(pr, golden[key + "_peer_rank"])
        np.testing.assert_array_equal(pt, golden[key + "_peer_token_idx"])
        np.testing.assert_array_equal(nt, golden[key + "_num_tokens"])
        np.testing.assert_array_equal(tpe, golden[key + "_tokens_per_expert"])


@pytest.mark.parametrize("R,T,K,E_l,factor,pattern", [
    (1, 1024, 2, 8, 2, "random"),          # c1
    (8, 16384, 8, 32, 4, "random"),        # c2: 16384 tokens/rank, 256 experts, top-8
    (8, 16384, 8, 16, 8, "skew"),          # c4: Zipf routing, capacity multiplier 1.0
    (2, 4096, 6, 32, 2, "random"),         # c5 at EP=2
    (1, 4096, 6, 64, 2, "random"),
    (4, 512, 1, 300, 152, "random"),       # many local experts, nearly all padding
    (3, 768, 5, 7, 2, "random"),           # odd sizes
])
def test_schedule_bit_exact_vs_oracle_full_size(mods, R, T, K, E_l, factor, pattern):
    _C, ops = mods
    topk = G.schedule_topk(R, T, K, E_l, pattern, seed=3)
    rank = R - 1
    C = T * K * factor
    ref = O.schedule(topk, E_l, C, rank)
    got, code = run_schedule(ops, _C, topk, E_l, C, rank)
    assert code == 0
    for a, b in zip(ref, got):
        np.testing.assert_array_equal(a, b)
    # size-independent properties: every route to a local expert appears exactly once, segments are sorted by expert
    pr, pt = got[0], got[1]
    n = int(got[2][0])
    real = pr[:n] >= 0
    keys = pr[:n][real].astype(np.int64) * (T * K) + pt[:n][real]
    assert np.unique(keys).size == keys.size
    local = topk.reshape(R, -1) - rank * E_l
    assert keys.size == int(((local >= 0) & (local < E_l)).sum())
    assert (pr[n:] == -1).all()


def test_schedule_overflow_sets_status_and_does_not_write(mods):
    _C, ops = mods
    topk = np.zeros((4, 512, 1), np.int32)          # every route of every rank to expert 0
    (pr, pt, nt, tpe), code = run_schedule(ops, _C, topk, 1, 512, 0)
    assert code == _C.ST_SCHEDULE_OVERFLOW
    assert int(nt[0]) == 2048 and (pr == -1).all()


def test_schedule_rejects_bad_arguments(mods):
    _C, ops = mods
    t = torch.zeros(1, 512, 2, dtype=torch.int32, device="cuda")
    for args in ((t, 0, 2048, 0), (t, 4, 1000, 0), (t, 4, 512, 0), (t, 4, 2048, 1), (t[0], 4, 2048, 0)):
        with pytest.raises(ValueError):
            ops.schedule(*args)


# ------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("name", ["q2d", "q3d", "qwide"])
def test_quantiser_byte_exact_vs_golden(mods, golden, name):
    _C, ops = mods
    x = bf16(golden[name + "_in"]).cuda()
    q, s, qt, st = ops.mxfp8_quantize(x, True, True)
    np.testing.assert_array_equal(q.view(torch.uint8).cpu().numpy(), golden[name + "_fp8"])
    np.testing.assert_array_equal(s.cpu().numpy(), golden[name + "_sc"])
    np.testing.assert_array_equal(qt.view(torch.uint8).cpu().numpy(), golden[name + "_fp8_t"])
    np.testing.assert_array_equal(st.cpu().numpy(), golden[name + "_sc_t"])
    q2, s2, none_a, none_b = ops.mxfp8_quantize(x, True, False)
    assert none_a is None and none_b is None and torch.equal(q2.view(torch.uint8), q.view(torch.uint8))


def test_quantiser_byte_exact_vs_oracle_large_and_edge_values(mods):
    _C, ops = mods
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(4, 256, 384, generator=g) * torch.exp(torch.randn(4, 256, 1, generator=g) * 4)).to(torch.bfloat16)
    x[0, :3] = 0                      # all-zero blocks
    x[1, 5, :32] = 448.0              # exactly representable maximum
    x[2, 7, 0] = 3.0e38               # huge
    x[3, 9, :64] = 1e-30              # tiny
    ref = O.mxfp8_quantize(x, True, True)
    got = ops.mxfp8_quantize(x.cuda(), True, True)
    for a, b in zip(ref, got):
        assert torch.equal(a.view(torch.uint8), b.cpu().view(torch.uint8))


# ------------------------------------------------------------------ element-wise
def test_epilogues_vs_oracle_and_known_answer(mods):
    _C, ops = mods
    g = torch.Generator().manual_seed(1)
    T, H, K = 768, 512, 6
    y = torch.randn(T, H, generator=g).to(torch.bfloat16)
    comb = torch.randn(T * K, H, generator=g).to(torch.bfloat16)
    w = torch.softmax(torch.randn(T, K, generator=g), -1)
    got = ops.fwd_epilogue(y.cuda(), comb.cuda(), w.cuda())
    assert_close("fwd_epilogue", O.fwd_epilogue(y, comb, w), got, (0.02, 1e-3))
    got = ops.bwd_epilogue(y.cuda(), comb.cuda())
    assert_close("bwd_epilogue", O.bwd_epilogue(y, comb), got, (0.04, 1e-3))
    # constants: shared = 1, routed = 2, w = 0.25, K = 1 -> 1.5 forward, 3.0 backward; >65535 tokens
    T = 66048
    one = torch.ones(T, 256, dtype=torch.bfloat16, device="cuda")
    two = one * 2
    w = torch.full((T, 1), 0.25, device="cuda")
    assert torch.all(ops.fwd_epilogue(one, two, w) == 1.5)
    assert torch.all(ops.bwd_epilogue(one, two) == 3.0)


@pytest.mark.parametrize("limit", [None, 4.0, 0.0])
def test_swiglu_fwd_bwd_vs_oracle(mods, limit):
    _C, ops = mods
    g = torch.Generator().manual_seed(2)
    rows, cols = 640, 384
    gate = (torch.randn(rows, cols, generator=g) * 3).to(torch.bfloat16)
    up = (torch.randn(rows, cols, generator=g) * 3).to(torch.bfloat16)
    dh = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    w = torch.rand(rows, generator=g) + 0.05
    w[::7] = 0.0
    n = torch.tensor([512], dtype=torch.int32, device="cuda")
    h = _C.swiglu_fwd(gate.cuda(), up.cuda(), limit, n)
    assert_close("hidden", O.swiglu_fwd(gate, up, limit)[:512], h[:512], (0.05, 2e-3))
    dg, du, rg = _C.swiglu_bwd(gate.cuda(), up.cuda(), dh.cuda(), limit, w.cuda(), True, n)
    rdg, rdu, hid = O.swiglu_bwd(gate, up, dh, limit)
    assert_close("d_gate", rdg[:512], dg[:512], (0.1, 2e-3))
    assert_close("d_up", rdu[:512], du[:512], (0.1, 2e-3))
    inv = torch.where(w > 0, 1 / w, torch.zeros_like(w))
    ref_rg = (dh.float() * inv[:, None] * hid).sum(1)
    assert_close("row_grad", ref_rg[:512], rg[:512], (0.05 * float(ref_rg.abs().max()), 1e-3))


# ------------------------------------------------------------------ dispatch / combine (EP = 1 path of the peer kernels)
def test_dispatch_and_combine_rows_single_rank(mods):
    _C, ops = mods
    g = torch.Generator().manual_seed(4)
    T, K, H, E = 512, 4, 512, 8
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    topk = torch.topk(torch.randn(T, E, generator=g), K).indices.to(torch.int32).numpy()[None]
    pr, pt, nt, tpe = O.schedule(topk, E, T * K * 2, 0)
    N = int(nt[0])
    prd, ptd, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, nt))
    MB = T * K * 2
    out = torch.full((MB, H), 7.0, dtype=torch.bfloat16, device="cuda")
    _C.dispatch_rows([x.data_ptr()], prd, ptd, ntd, MB, K, H, out)
    ref = torch.zeros(N, H, dtype=torch.bfloat16)
    real = pr[:N] >= 0
    ref[torch.from_numpy(real)] = x.cpu()[torch.from_numpy(pt[:N][real] // K).long()]
    assert torch.equal(out[:N].cpu(), ref)
    assert torch.all(out[N:] == 7.0)                    # rows past num_tokens are untouched
    # scaled variant
    w = torch.rand(T, K, generator=g).cuda()
    ws = torch.empty(MB, device="cuda")
    _C.dispatch_rows([x.data_ptr()], prd, ptd, ntd, MB, K, H, out, [w.data_ptr()], ws)
    wrow = torch.zeros(N)
    wrow[torch.from_numpy(real)] = w.cpu().reshape(-1)[torch.from_numpy(pt[:N][real]).long()]
    assert torch.equal(ws[:N].cpu(), wrow)
    assert torch.equal(out[:N].cpu(), (ref.float() * wrow[:, None]).to(torch.bfloat16))
    # combine is the inverse permutation
    comb = torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda")
    vals = torch.zeros(T * K, device="cuda")
    rowv = torch.arange(MB, dtype=torch.float32, device="cuda")
    _C.dispatch_rows([x.data_ptr()], prd, ptd, ntd, MB, K, H, out)
    _C.combine_rows(out, [comb.data_ptr()], prd, ptd, ntd, MB, H, rowv, [vals.data_ptr()])
    assert torch.equal(comb.view(T, K, H), x[:, None, :].expand(T, K, H))
    inv = torch.empty(T * K)
    inv[torch.from_numpy(pt[:N][real]).long()] = torch.arange(N, dtype=torch.float32)[torch.from_numpy(real)]
    assert torch.equal(vals.cpu(), inv)


def test_barrier_wait_is_bounded_and_reports_through_the_status_word(mods):
    # failure made on the host: a 2-rank pointer list whose second "rank" is a local word nobody signals from,
    # so this rank's own word only ever receives its own arrival.  The wait must give up and set the status.
    _C, ops = mods
    mine = torch.zeros(1, dtype=torch.int32, device="cuda")
    other = torch.zeros(1, dtype=torch.int32, device="cuda")
    target = torch.zeros(1, dtype=torch.int32, device="cuda")
    _C.set_barrier_timeout_ms(200)
    try:
        _C.barrier_all(mine, [mine.data_ptr(), other.data_ptr()], 0, target, rank=0)
        torch.cuda.synchronize()
        assert _C.check_status() == _C.ST_BARRIER_TIMEOUT
        assert int(target.item()) == 2 and int(mine.item()) == 1 and int(other.item()) == 1
        # the context is still usable and a complete barrier (both arrivals present) passes
        other2 = torch.zeros(1, dtype=torch.int32, device="cuda")
        mine.fill_(3)          # as if the peer had already arrived for the next round
        _C.barrier_all(mine, [mine.data_ptr(), other2.data_ptr()], 0, target, rank=0)
        torch.cuda.synchronize()
        assert _C.check_status() == 0
    finally:
        _C.set_barrier_timeout_ms(10000)


# ------------------------------------------------------------------ grouped GEMM, all four operand layouts
def _groups(rows_per_group):
    offs = np.concatenate([[0], np.cumsum(rows_per_group)]).astype(np.int32)
    gob = np.concatenate([np.full(n // 128, g, np.int32) for g, n in enumerate(rows_per_group)])
    return torch.from_numpy(offs).cuda(), torch.from_numpy(gob).cuda(), int(offs[-1])


@pytest.mark.parametrize("rows_per_group,N,K", [([256], 256, 64), ([256, 512, 0, 256], 512, 256), ([1024, 256], 256, 1024)])
def test_gemm_nt(mods, rows_per_group, N, K):
    _C, ops = mods
    offs, gob, rows = _groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(5)
    cap = rows + 256
    A = torch.randn(cap, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(G_, N, K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    D = torch.full((cap, N), 3.0, dtype=torch.bfloat16, device="cuda")
    n = torch.tensor([rows], dtype=torch.int32, device="cuda")
    gob_full = torch.cat([gob, torch.full((2,), -1, dtype=torch.int32, device="cuda")])
    _C.grouped_gemm(0, A, W, D, num_rows=n, group_of_block=gob_full, G=G_, N=N, K=K)
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        ref = (A[s:e].float() @ W[gi].float().T).to(torch.bfloat16)
        assert_close(f"nt group {gi}", ref, D[s:e], GEMM_TOL)
    assert torch.all(D[rows:] == 3.0)


def test_gemm_row_window_touches_only_its_rows(mods):
    _C, ops = mods
    rows_per_group, N, K = [512, 256, 768], 256, 128
    offs, gob, rows = _groups(rows_per_group)
    g = torch.Generator().manual_seed(15)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(3, N, K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    full = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(0, A, W, full, group_of_block=gob, G=3, N=N, K=K)
    n = torch.tensor([1280], dtype=torch.int32, device="cuda")      # fewer rows than the last window asks for
    part = torch.full((rows, N), 9.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(0, A, W, part, num_rows=n, group_of_block=gob, G=3, N=N, K=K, row_begin=256, row_end=768)
    _C.grouped_gemm(0, A, W, part, num_rows=n, group_of_block=gob, G=3, N=N, K=K, row_begin=1024, row_end=1536)
    assert _C.check_status() == 0
    assert torch.equal(part[256:768], full[256:768]) and torch.equal(part[1024:1280], full[1024:1280])
    assert torch.all(part[:256] == 9.0) and torch.all(part[768:1024] == 9.0) and torch.all(part[1280:] == 9.0)


@pytest.mark.parametrize("limit", [None, 1.0])
def test_gemm_swiglu(mods, limit):
    _C, ops = mods
    rows_per_group, N, K = [512, 256, 256], 384, 512
    offs, gob, rows = _groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(6)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16).cuda()
    Wg = (torch.randn(G_, N, K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    Wu = (torch.randn(G_, N, K, generator=g) * 0.1).to(torch.bfloat16).cuda()
    gate, up, hid = (torch.empty(rows, N, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    _C.grouped_gemm(1, A, Wg, gate, group_of_block=gob, G=G_, N=N, K=K, B2=Wu, D2=up, D3=hid, swiglu_limit=limit)
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        rg = (A[s:e].float() @ Wg[gi].float().T).to(torch.bfloat16)
        ru = (A[s:e].float() @ Wu[gi].float().T).to(torch.bfloat16)
        assert_close("gate", rg, gate[s:e], GEMM_TOL)
        assert_close("up", ru, up[s:e], GEMM_TOL)
        # hidden must be SwiGLU of the gate/up the kernel itself stored
        assert_close("hidden", O.swiglu_fwd(gate[s:e].cpu(), up[s:e].cpu(), limit), hid[s:e], (0.05, 2e-3))


@pytest.mark.parametrize("dual", [False, True])
@pytest.mark.parametrize("N", [256, 384])
def test_gemm_nn(mods, dual, N):
    _C, ops = mods
    rows_per_group, K = [256, 512], 256
    offs, gob, rows = _groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(7)
    A = torch.randn(rows, K, generator=g).to(torch.bfloat16).cuda()
    W = (torch.randn(G_, K, N, generator=g) * 0.1).to(torch.bfloat16).cuda()
    A2 = torch.randn(rows, K, generator=g).to(torch.bfloat16).cuda() if dual else None
    W2 = (torch.randn(G_, K, N, generator=g) * 0.1).to(torch.bfloat16).cuda() if dual else None
    D = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(2, A, W, D, group_of_block=gob, G=G_, N=N, K=K, A2=A2, B2=W2)
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        ref = A[s:e].float() @ W[gi].float()
        if dual:
            ref = ref + A2[s:e].float() @ W2[gi].float()
        assert_close(f"nn group {gi}", ref.to(torch.bfloat16), D[s:e], GEMM_TOL)


@pytest.mark.parametrize("rows_per_group,M,N", [([256], 128, 256), ([512, 0, 256], 256, 384), ([256, 1024], 384, 512)])
def test_gemm_wgrad(mods, rows_per_group, M, N):
    _C, ops = mods
    offs, gob, rows = _groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator().manual_seed(8)
    A = torch.randn(rows, M, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(rows, N, generator=g).to(torch.bfloat16).cuda()
    D = torch.full((G_, M, N), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(3, A, B, D, group_offsets=offs, G=G_, M=M, N=N)
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        ref = (A[s:e].float().T @ B[s:e].float()).to(torch.bfloat16)
        tol = (GEMM_TOL[0] * 8, GEMM_TOL[1]) if e > s else (0.0, 0.0)
        assert_close(f"wgrad group {gi}", ref, D[gi], tol) if e > s else None
        if e == s:
            assert torch.all(D[gi] == 0)


def test_gemm_wgrad_leaves_out_the_padding_rows_it_is_told_about(mods):
    """group_k_end: rows of a group from there on are padding (zero in both operands).  The kernel stops at the next
    multiple of 64 rows, so whatever lies beyond that -- NaN here -- must not reach the result."""
    _C, ops = mods
    rows_per_group, M, N = [512, 768, 0, 256], 256, 384
    real = [300, 520, 0, 256]
    offs, gob, rows = _groups(rows_per_group)
    g = torch.Generator().manual_seed(18)
    A = torch.randn(rows, M, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(rows, N, generator=g).to(torch.bfloat16).cuda()
    o = offs.cpu().numpy()
    k_end = torch.tensor([int(o[i]) + real[i] for i in range(4)], dtype=torch.int32, device="cuda")
    for i in range(4):
        s, e = int(o[i]) + real[i], int(o[i + 1])
        A[s:e] = 0
        B[s:e] = 0
        s64 = int(o[i]) + (real[i] + 63) // 64 * 64
        A[s64:e] = float("nan")
        B[s64:e] = float("nan")
    D = torch.full((4, M, N), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(3, A, B, D, group_offsets=offs, G=4, M=M, N=N, group_k_end=k_end)
    assert _C.check_status() == 0
    for i in range(4):
        s, e = int(o[i]), int(o[i]) + real[i]
        if real[i] == 0:
            assert torch.all(D[i] == 0)
            continue
        ref = (A[s:e].float().T @ B[s:e].float()).to(torch.bfloat16)
        assert_close(f"wgrad group {i}", ref, D[i], (GEMM_TOL[0] * 8, GEMM_TOL[1]))
