"""The persistent forward GEMM (mode 4 of mokb_grouped_gemm_bf16: gate/up + SwiGLU and the down projection of the same
rows in one launch) and the counters that tie it to dispatch and combine launches running beside it.  The reference
synchronises the tasks of its megakernel the same way (csrc/megakernel/utils.cuh:1-13, forward.cuh:146-266), without
a time limit; here every wait gives up after 2 s with a status code, which the last two tests make happen on purpose
by leaving a counter untouched (nothing faults or hangs: the kernels return and the context stays usable)."""
import pytest
import torch

from tests.gpu_common import groups

pytestmark = pytest.mark.gpu


def problem(rows_per_group, H, I, seed=70):
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    g = torch.Generator(device="cuda").manual_seed(seed)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)
    return dict(rows=rows, G=G_, gob=gob, x=rnd(rows, H), Wg=rnd(G_, I, H, scale=0.05), Wu=rnd(G_, I, H, scale=0.05),
                Wd=rnd(G_, H, I, scale=0.05), H=H, I=I)


def outputs(p, fill=None):
    mk = (lambda *s: torch.full(s, fill, dtype=torch.bfloat16, device="cuda")) if fill is not None else \
         (lambda *s: torch.empty(*s, dtype=torch.bfloat16, device="cuda"))
    return mk(p["rows"], p["I"]), mk(p["rows"], p["I"]), mk(p["rows"], p["I"]), mk(p["rows"], p["H"])


def separate(_C, p, limit=None):
    gate, up, hid, y = outputs(p)
    _C.grouped_gemm(1, p["x"], p["Wg"], gate, group_of_block=p["gob"], G=p["G"], N=p["I"], K=p["H"], B2=p["Wu"], D2=up, D3=hid,
                    swiglu_limit=limit)
    _C.grouped_gemm(0, hid, p["Wd"], y, group_of_block=p["gob"], G=p["G"], N=p["H"], K=p["I"])
    return gate, up, hid, y


@pytest.mark.parametrize("rows_per_group,H,I,window,limit", [
    ([512, 256, 0, 768], 512, 384, 512, None),        # three windows, I = 3 * 128
    ([256, 1280], 1024, 256, 0, 1.5),                 # one window, clamped
    ([2048, 512, 3072], 768, 512, 1024, None),        # more tiles than CTA pairs: every pair walks both kinds of tile
])
def test_fused_forward_gemm_equals_the_two_launches_bit_for_bit(rows_per_group, H, I, window, limit):
    from mok import _C
    p = problem(rows_per_group, H, I)
    ref = separate(_C, p, limit)
    gate, up, hid, y = outputs(p, fill=3.0)
    n = torch.tensor([p["rows"] - 256], dtype=torch.int32, device="cuda")      # the last 256-row block is not scheduled
    blk = torch.zeros(p["rows"] // 256, dtype=torch.int32, device="cuda")
    nwin = (p["rows"] + window - 1) // window if window else 1
    done = torch.zeros(nwin, dtype=torch.int32, device="cuda")
    _C.grouped_gemm(4, p["x"], p["Wg"], gate, num_rows=n, group_of_block=p["gob"], G=p["G"], N=I, K=H, B2=p["Wu"], D2=up, D3=hid,
                    B3=p["Wd"], D4=y, N2=H, window_rows=window, blk_done=blk, win_done=done, swiglu_limit=limit)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    live = p["rows"] - 256
    for name, a, b in zip(("gate", "up", "hidden", "y"), ref, (gate, up, hid, y)):
        assert torch.equal(a[:live], b[:live]), name
        assert torch.all(b[live:] == 3.0), f"{name}: rows past num_rows were written"
    # the counters: 8 epilogue warps per tile
    assert blk[: live // 256].tolist() == [I // 128 * 8] * (live // 256) and blk[live // 256:].sum().item() == 0
    w = window or p["rows"]
    want = [max(0, min(live, (c + 1) * w) - c * w) // 256 * (H // 256) * 8 for c in range(nwin)]
    assert done.tolist() == want


def test_fused_forward_gemm_without_the_down_projection():
    from mok import _C
    p = problem([512, 768], 512, 256, seed=71)
    ref = separate(_C, p)
    gate, up, hid, _ = outputs(p)
    blk = torch.zeros(p["rows"] // 256, dtype=torch.int32, device="cuda")
    _C.grouped_gemm(4, p["x"], p["Wg"], gate, group_of_block=p["gob"], G=p["G"], N=256, K=512, B2=p["Wu"], D2=up, D3=hid, blk_done=blk)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    assert all(torch.equal(a, b) for a, b in zip(ref[:3], (gate, up, hid)))


def test_dispatch_counter_feeds_the_gemm_and_the_gemm_counter_feeds_combine():
    """dispatch (side stream) -> fused GEMM (this stream) -> combine (second side stream), ordered only by counters:
    the three launches may run in any order or at once."""
    from mok import _C
    T, K, H, I, E = 1024, 2, 512, 256, 4
    g = torch.Generator().manual_seed(72)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    from oracle import mok_oracle as O
    topk = torch.topk(torch.randn(T, E, generator=g), K).indices.to(torch.int32).numpy()[None]
    C = T * K * 2
    pr, pt, nt, tpe = O.schedule(topk, E, C, 0)
    N = int(nt[0])
    prd, ptd, ntd = (torch.from_numpy(a).cuda() for a in (pr, pt, nt))
    gob = torch.repeat_interleave(torch.arange(E, dtype=torch.int32), torch.from_numpy(tpe // 128).long())
    gob = torch.cat([gob, torch.full((C // 128 - gob.numel(),), -1, dtype=torch.int32)]).cuda()
    gd = torch.Generator(device="cuda").manual_seed(73)
    rnd = lambda *shape: (torch.randn(*shape, generator=gd, device="cuda") * 0.05).to(torch.bfloat16)
    Wg, Wu, Wd = rnd(E, I, H), rnd(E, I, H), rnd(E, H, I)
    window, blocks = 512, 24
    nwin = C // window
    # reference: everything in stream order
    xr = torch.zeros(C, H, dtype=torch.bfloat16, device="cuda")
    _C.dispatch_rows([x.data_ptr()], prd, ptd, ntd, C, K, H, xr)
    p = dict(rows=C, G=E, gob=gob, x=xr, Wg=Wg, Wu=Wu, Wd=Wd, H=H, I=I)
    gate0, up0, hid0, y0 = outputs(p)
    _C.grouped_gemm(1, xr, Wg, gate0, num_rows=ntd, group_of_block=gob, G=E, N=I, K=H, B2=Wu, D2=up0, D3=hid0)
    _C.grouped_gemm(0, hid0, Wd, y0, num_rows=ntd, group_of_block=gob, G=E, N=H, K=I)
    comb0 = torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda")
    _C.combine_rows(y0, [comb0.data_ptr()], prd, ptd, ntd, C, H)
    torch.cuda.synchronize()
    # counters only
    ready = torch.zeros(nwin, dtype=torch.int32, device="cuda")
    done = torch.zeros(nwin, dtype=torch.int32, device="cuda")
    blk = torch.zeros(C // 256, dtype=torch.int32, device="cuda")
    xr1 = torch.full((C, H), 9.0, dtype=torch.bfloat16, device="cuda")
    gate, up, hid, y = outputs(p)
    comb = torch.zeros(T * K, H, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(s_out):          # enqueued first: it has to wait for the GEMM, which has to wait for the dispatch
        for c in range(nwin):
            _C.combine_rows_window(y, [comb.data_ptr()], prd, ptd, ntd, C, c * window, (c + 1) * window, H, blocks=blocks,
                                   wait_counter=done[c:], arrivals_per_row_block=H // 256 * 8)
    _C.grouped_gemm(4, xr1, Wg, gate, num_rows=ntd, group_of_block=gob, G=E, N=I, K=H, B2=Wu, D2=up, D3=hid, B3=Wd, D4=y, N2=H,
                    window_rows=window, win_ready=ready, win_ready_target=blocks, blk_done=blk, win_done=done)
    with torch.cuda.stream(s_in):
        for c in range(nwin):
            _C.dispatch_rows_window([x.data_ptr()], prd, ptd, ntd, C, c * window, (c + 1) * window, K, H, xr1, blocks=blocks,
                                    done_counter=ready[c:])
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    live_windows = (N + window - 1) // window
    assert ready[:live_windows].tolist() == [blocks] * live_windows
    assert torch.equal(xr1[:N], xr[:N]) and torch.equal(y[:N], y0[:N]) and torch.equal(hid[:N], hid0[:N])
    assert torch.equal(comb, comb0)


def test_a_gemm_whose_window_never_becomes_ready_gives_up_with_a_status_code():
    from mok import _C
    p = problem([512, 512], 256, 128, seed=74)
    gate, up, hid, y = outputs(p, fill=5.0)
    ready = torch.zeros(2, dtype=torch.int32, device="cuda")
    ready[0] = 4                                  # window 0 is ready, window 1 never will be
    blk = torch.zeros(p["rows"] // 256, dtype=torch.int32, device="cuda")
    _C.grouped_gemm(4, p["x"], p["Wg"], gate, group_of_block=p["gob"], G=2, N=128, K=256, B2=p["Wu"], D2=up, D3=hid, B3=p["Wd"], D4=y,
                    N2=256, window_rows=512, win_ready=ready, win_ready_target=4, blk_done=blk)
    torch.cuda.synchronize()
    assert _C.check_status() == _C.ST_FLAG_TIMEOUT
    assert torch.all(gate[512:] == 5.0) and torch.all(y[512:] == 5.0)          # nothing of window 1 was computed
    # the context is still usable, and the same call with both windows ready completes
    ready.fill_(4)
    blk.zero_()
    _C.grouped_gemm(4, p["x"], p["Wg"], gate, group_of_block=p["gob"], G=2, N=128, K=256, B2=p["Wu"], D2=up, D3=hid, B3=p["Wd"], D4=y,
                    N2=256, window_rows=512, win_ready=ready, win_ready_target=4, blk_done=blk)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    ref = separate(_C, p)
    assert all(torch.equal(a, b) for a, b in zip(ref, (gate, up, hid, y)))


def test_a_combine_whose_rows_never_arrive_gives_up_and_copies_nothing():
    from mok import _C
    rows, H = 512, 256
    src = torch.ones(rows, H, dtype=torch.bfloat16, device="cuda")
    dst = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
    pr = torch.zeros(rows, dtype=torch.int32, device="cuda")
    pt = torch.arange(rows, dtype=torch.int32, device="cuda")
    n = torch.tensor([rows], dtype=torch.int32, device="cuda")
    counter = torch.tensor([7], dtype=torch.int32, device="cuda")            # 2 row blocks x 8 arrivals = 16 are needed
    _C.combine_rows_window(src, [dst.data_ptr()], pr, pt, n, rows, 0, rows, H, blocks=4, wait_counter=counter, arrivals_per_row_block=8)
    torch.cuda.synchronize()
    assert _C.check_status() == _C.ST_FLAG_TIMEOUT and torch.all(dst == 0)
    counter.fill_(16)
    _C.combine_rows_window(src, [dst.data_ptr()], pr, pt, n, rows, 0, rows, H, blocks=4, wait_counter=counter, arrivals_per_row_block=8)
    torch.cuda.synchronize()
    assert _C.check_status() == 0 and torch.all(dst == 1)
