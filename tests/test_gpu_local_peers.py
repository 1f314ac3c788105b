"""The multi-rank branches of the communication kernels on ONE GPU: every "peer" is a distinct local buffer, so the
pointer lists have ep_size > 1 entries and rows really come from / go to ranks other than the caller's, while all
loads and stores stay on this device.  The schedule is the oracle's for R ranks; each rank's call is made in turn
(the kernels never wait on one another).  Reference tests: tests/test_ops.py:95-102 (route all-gather, exact),
:173-226 (schedule), tests/test_functional_e2e.py (dispatch / combine through the layer)."""
import numpy as np
import pytest
import torch

from oracle import mok_oracle as O

pytestmark = pytest.mark.gpu


def make_routes(R, T, K, E_l, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(R, T, E_l * R, generator=g)
    return torch.topk(logits, K, dim=2).indices.to(torch.int32).numpy()


@pytest.mark.parametrize("R,T,K", [(2, 512, 2), (4, 768, 3), (8, 512, 8)])
def test_all_gather_top_experts_over_local_peers(R, T, K):
    from mok import _C
    routes = make_routes(R, T, K, 4, seed=50 + R)
    bufs = [torch.full((R, T, K), -7, dtype=torch.int32, device="cuda") for _ in range(R)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(R):
        _C.all_gather_top_experts(torch.from_numpy(routes[r]).cuda(), bufs[r], 0, r, 2048, ptrs)
    torch.cuda.synchronize()
    want = torch.from_numpy(routes)
    for r in range(R):
        assert torch.equal(bufs[r].cpu(), want), f"rank {r}'s gathered routes differ"


@pytest.mark.parametrize("R,T,K,H,E_l", [(2, 512, 2, 512, 4), (4, 512, 4, 256, 3), (8, 512, 8, 1024, 2)])
def test_dispatch_and_combine_over_local_peers(R, T, K, H, E_l):
    from mok import _C
    routes = make_routes(R, T, K, E_l, seed=60 + R)
    g = torch.Generator().manual_seed(61)
    x = [torch.randn(T, H, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
    w = [torch.rand(T, K, generator=g).cuda() for _ in range(R)]
    x_ptrs, w_ptrs = [t.data_ptr() for t in x], [t.data_ptr() for t in w]
    comb = [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    vals = [torch.full((T * K,), -1.0, device="cuda") for _ in range(R)]
    comb_ptrs, val_ptrs = [t.data_ptr() for t in comb], [t.data_ptr() for t in vals]
    C = T * K * R
    x_all = torch.stack([t.cpu() for t in x])                       # [R, T, H]
    w_all = torch.stack([t.cpu() for t in w]).reshape(R, T * K)
    owner_row = [torch.full((T * K,), -1.0) for _ in range(R)]      # expected row_values per home rank
    remote_rows = 0
    for q in range(R):                                              # rank q owns experts [q*E_l, (q+1)*E_l)
        pr, pt, nt, tpe = O.schedule(routes, E_l, C, q)
        N = int(nt[0])
        real = torch.from_numpy(pr[:N] >= 0)
        prt, ptt = torch.from_numpy(pr[:N]).long(), torch.from_numpy(pt[:N]).long()
        remote_rows += int(((prt >= 0) & (prt != q)).sum())
        prd, ptd, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, nt))
        out = torch.full((C, H), 7.0, dtype=torch.bfloat16, device="cuda")
        _C.dispatch_rows(x_ptrs, prd, ptd, ntd, C, K, H, out)
        ref = torch.zeros(N, H, dtype=torch.bfloat16)
        ref[real] = x_all[prt[real], ptt[real] // K]
        assert torch.equal(out[:N].cpu(), ref), f"owner {q}: pulled rows differ"
        assert torch.all(out[N:] == 7.0)
        # scaled pull: row * router weight of its route in fp32, rounded to bf16; the weight itself comes along
        scaled = torch.empty(C, H, dtype=torch.bfloat16, device="cuda")
        wrow = torch.empty(C, device="cuda")
        _C.dispatch_rows(x_ptrs, prd, ptd, ntd, C, K, H, scaled, w_ptrs, wrow)
        wref = torch.zeros(N)
        wref[real] = w_all[prt[real], ptt[real]]
        assert torch.equal(wrow[:N].cpu(), wref), f"owner {q}: router weights differ"
        assert torch.equal(scaled[:N].cpu(), (ref.float() * wref[:, None]).to(torch.bfloat16))
        # push the pulled rows home, with the row number as the per-route value
        rowv = torch.arange(C, dtype=torch.float32, device="cuda") + 1000.0 * q
        _C.combine_rows(out, comb_ptrs, prd, ptd, ntd, C, H, rowv, val_ptrs)
        for r in range(R):
            sel = real & (prt == r)
            owner_row[r][ptt[sel]] = torch.arange(N, dtype=torch.float32)[sel] + 1000.0 * q
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    assert remote_rows > 0
    for r in range(R):      # every route of every home rank came back to slot t*K+k, from whichever rank owns its expert
        assert torch.equal(comb[r].view(T, K, H), x[r][:, None, :].expand(T, K, H)), f"home rank {r}: combine buffer differs"
        assert torch.equal(vals[r].cpu(), owner_row[r]), f"home rank {r}: per-route values differ"


@pytest.mark.parametrize("R,T,K,H,I,E_l", [(4, 512, 2, 512, 256, 2), (8, 512, 4, 256, 384, 1)])
def test_gemm_epilogue_pushes_rows_to_local_peers_like_a_combine_launch(R, T, K, H, I, E_l):
    """The down projection (mode 0, and as the second phase of mode 4) and the dual input gradient (mode 2) with their
    rows pushed to the home ranks' buffers from the epilogue: bit for bit what the plain GEMM followed by combine_rows
    leaves there, including the per-route value that travels with the input gradient."""
    from mok import _C
    routes = make_routes(R, T, K, E_l, seed=80 + R)
    q = R - 1                                                      # the rank whose experts we run
    C = T * K * R
    pr, pt, nt, tpe = O.schedule(routes, E_l, C, q)
    N = int(nt[0])
    prd, ptd, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, nt))
    gob = torch.repeat_interleave(torch.arange(E_l, dtype=torch.int32), torch.from_numpy(tpe // 128).long())
    gob = torch.cat([gob, torch.full((C // 128 - gob.numel(),), -1, dtype=torch.int32)]).cuda()
    gd = torch.Generator(device="cuda").manual_seed(81)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=gd, device="cuda") * scale).to(torch.bfloat16)
    hid, Wd = rnd(C, I), rnd(E_l, H, I, scale=0.05)
    x, Wg, Wu = rnd(C, H), rnd(E_l, I, H, scale=0.05), rnd(E_l, I, H, scale=0.05)
    dg, du = rnd(C, I), rnd(C, I)
    rowv = torch.arange(C, dtype=torch.float32, device="cuda") * 0.5
    zeros = lambda: [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    ptrs = lambda ts: [t.data_ptr() for t in ts]

    # reference: GEMM into a local buffer, then the combine kernel
    y = torch.empty(C, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(0, hid, Wd, y, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I)
    want = zeros()
    _C.combine_rows(y, ptrs(want), prd, ptd, ntd, C, H)
    dx = torch.empty(C, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(2, dg, Wg, dx, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I, A2=du, B2=Wu)
    want_dx, want_val = zeros(), [torch.full((T * K,), -1.0, device="cuda") for _ in range(R)]
    _C.combine_rows(dx, ptrs(want_dx), prd, ptd, ntd, C, H, rowv, ptrs(want_val))

    # mode 0, pushed only (no local copy)
    got = zeros()
    _C.grouped_gemm(0, hid, Wd, None, rows=C, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I, ldd=H,
                    push_ptrs=ptrs(got), push_rank=prd, push_idx=ptd)
    # mode 2 with a second operand pair, a local copy and the per-route values
    got_dx, got_val = zeros(), [torch.full((T * K,), -1.0, device="cuda") for _ in range(R)]
    dx2 = torch.full((C, H), 3.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(2, dg, Wg, dx2, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I, A2=du, B2=Wu,
                    push_ptrs=ptrs(got_dx), push_rank=prd, push_idx=ptd, push_values=rowv, push_value_ptrs=ptrs(got_val))
    # mode 4: gate/up + SwiGLU + down, the down rows pushed only
    gate, up, hid4 = (torch.empty(C, I, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    blk = torch.zeros(C // 256, dtype=torch.int32, device="cuda")
    got4 = zeros()
    _C.grouped_gemm(4, x, Wg, gate, num_rows=ntd, group_of_block=gob, G=E_l, N=I, K=H, B2=Wu, D2=up, D3=hid4, B3=Wd, N2=H,
                    window_rows=512, blk_done=blk, push_ptrs=ptrs(got4), push_rank=prd, push_idx=ptd)
    y4 = torch.empty(C, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(0, hid4, Wd, y4, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I)
    want4 = zeros()
    _C.combine_rows(y4, ptrs(want4), prd, ptd, ntd, C, H)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    assert int(((torch.from_numpy(pr[:N]) >= 0) & (torch.from_numpy(pr[:N]) != q)).sum()) > 0
    for r in range(R):
        assert torch.equal(got[r], want[r]), f"mode 0: rank {r}'s buffer differs"
        assert torch.equal(got_dx[r], want_dx[r]) and torch.equal(got_val[r], want_val[r]), f"mode 2: rank {r}'s buffers differ"
        assert torch.equal(got4[r], want4[r]), f"mode 4: rank {r}'s buffer differs"
    assert torch.equal(dx2[:N], dx[:N]) and torch.all(dx2[N:] == 3.0)


@pytest.mark.parametrize("R,T,K,H,scaled", [(2, 512, 2, 256, False), (4, 512, 4, 512, True), (2, 512, 2, 7168, True)])
def test_dispatch_quantises_the_rows_it_pulls_like_the_quantiser(R, T, K, H, scaled):
    """The pull's row-wise MXFP8 output (from the registers the row passes through) against the quantiser kernel run
    on the pulled bf16 rows: bytes and scales identical, padding rows included; hidden 256 is the case where only half
    of a warp's lanes hold data."""
    from mok import _C, ops
    E_l = 2
    routes = make_routes(R, T, K, E_l, seed=90 + R)
    g = torch.Generator().manual_seed(91)
    x = [(torch.randn(T, H, generator=g) * torch.exp(torch.randn(T, 1, generator=g) * 2)).to(torch.bfloat16).cuda() for _ in range(R)]
    w = [torch.rand(T, K, generator=g).cuda() for _ in range(R)]
    C = T * K * R
    pr, pt, nt, tpe = O.schedule(routes, E_l, C, R - 1)
    N = int(nt[0])
    prd, ptd, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, nt))
    out = torch.zeros(C, H, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(C, H, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(C // 128, H // 128, 32, 16, dtype=torch.uint8, device="cuda")
    wrow = torch.empty(C, device="cuda") if scaled else None
    _C.dispatch_rows_window([t.data_ptr() for t in x], prd, ptd, ntd, C, 0, C, K, H, out,
                            [t.data_ptr() for t in w] if scaled else None, wrow, blocks=32, q_out=q, q_sc_out=sc)
    torch.cuda.synchronize()
    live = (N + 127) // 128 * 128
    ref_q, ref_s, _, _ = ops.mxfp8_quantize(out[:live].contiguous(), True, False)
    assert torch.equal(q[:N], ref_q.view(torch.uint8)[:N])
    assert torch.equal(O.unpack_scales(sc.cpu())[:N], O.unpack_scales(ref_s.cpu())[:N])
    assert int((torch.from_numpy(pr[:N]) < 0).sum()) > 0          # the case has padding rows


def test_transposed_only_quantiser_matches_the_two_way_quantiser():
    from mok import ops
    g = torch.Generator().manual_seed(92)
    x = (torch.randn(384, 640, generator=g) * torch.exp(torch.randn(384, 1, generator=g) * 3)).to(torch.bfloat16).cuda()
    x[5] = 0
    _, _, qt, st = ops.mxfp8_quantize(x, True, True)
    n1, n2, qt2, st2 = ops.mxfp8_quantize(x, False, True)       # the column-only kernel (128 x 64 tiles)
    assert n1 is None and n2 is None
    assert torch.equal(qt.view(torch.uint8), qt2.view(torch.uint8)) and torch.equal(st, st2)


def test_a_route_index_outside_the_buffers_is_skipped_and_reported():
    """A schedule entry that names a route outside [0, tokens * topk) -- a stale or foreign schedule -- must not become
    an access outside a peer's buffer: the pull writes a zero row, the push kernels and the GEMM epilogue store nothing
    for that row, every other row is as without the bad entry, and the status words name the kernel kind, the row and
    the index."""
    from mok import _C
    R, T, K, H, I, E_l = 2, 512, 2, 256, 256, 2
    routes = make_routes(R, T, K, E_l, seed=95)
    C = T * K * R
    pr, pt, nt, tpe = O.schedule(routes, E_l, C, 1)
    N = int(nt[0])
    live = np.flatnonzero(pr[:N] >= 0)
    bad_row, bad_idx = int(live[len(live) // 2]), T * K + 12345
    pt_bad = pt.copy()
    pt_bad[bad_row] = bad_idx
    prd, ptd, ptb, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, pt_bad, nt))
    g = torch.Generator().manual_seed(96)
    x = [torch.randn(T, H, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
    ptrs = lambda ts: [t.data_ptr() for t in ts]

    def expect(kind):
        torch.cuda.synchronize()
        assert _C.check_status() == _C.ST_BAD_INDEX
        assert _C.status_detail() == [_C.ST_BAD_INDEX, kind, bad_row, bad_idx]

    # pull
    good = torch.zeros(C, H, dtype=torch.bfloat16, device="cuda")
    _C.dispatch_rows_window(ptrs(x), prd, ptd, ntd, C, 0, C, K, H, good, index_limit=T * K)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    got = torch.full((C, H), 7.0, dtype=torch.bfloat16, device="cuda")
    _C.dispatch_rows_window(ptrs(x), prd, ptb, ntd, C, 0, C, K, H, got, index_limit=T * K)
    expect(1)
    keep = torch.ones(N, dtype=torch.bool, device="cuda")
    keep[bad_row] = False
    assert torch.equal(got[:N][keep], good[:N][keep]) and torch.all(got[bad_row] == 0)

    # push kernel
    want = [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    _C.combine_rows_window(good, ptrs(want), prd, ptd, ntd, C, 0, C, H, index_limit=T * K)
    home, slot = int(pr[bad_row]), int(pt[bad_row])
    want[home][slot] = 0                                           # the one row that must stay untouched
    out = [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    _C.combine_rows_window(good, ptrs(out), prd, ptb, ntd, C, 0, C, H, index_limit=T * K)
    expect(2)
    assert all(torch.equal(a, b) for a, b in zip(out, want))

    # GEMM epilogue push (BF16 down projection)
    gob = torch.repeat_interleave(torch.arange(E_l, dtype=torch.int32), torch.from_numpy(tpe // 128).long())
    gob = torch.cat([gob, torch.full((C // 128 - gob.numel(),), -1, dtype=torch.int32)]).cuda()
    gd = torch.Generator(device="cuda").manual_seed(97)
    hid = (torch.randn(C, I, generator=gd, device="cuda")).to(torch.bfloat16)
    Wd = (torch.randn(E_l, H, I, generator=gd, device="cuda") * 0.05).to(torch.bfloat16)
    ref = [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    _C.grouped_gemm(0, hid, Wd, None, rows=C, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I, ldd=H,
                    push_ptrs=ptrs(ref), push_rank=prd, push_idx=ptd, push_index_limit=T * K)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    ref[home][slot] = 0
    out = [torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    _C.grouped_gemm(0, hid, Wd, None, rows=C, num_rows=ntd, group_of_block=gob, G=E_l, N=H, K=I, ldd=H,
                    push_ptrs=ptrs(out), push_rank=prd, push_idx=ptb, push_index_limit=T * K)
    expect(3)
    assert all(torch.equal(a, b) for a, b in zip(out, ref))
