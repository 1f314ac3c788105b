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
