"""The schedule entry point for callers that cannot allocate device memory
(mokb_schedule_noalloc): it must give the same schedule, bit for bit, as mokb_schedule.

Who needs it: code that runs where cudaMalloc is not available to it -- under a host
framework that owns the device heap, inside a step loop that must not hit cudaMalloc's
implicit device synchronisation, or in a process that fixes its memory at start-up.  The
work area is one array inside the library that every call shares and that keeps the last
call's contents, so the test makes two calls in a row, the second on a different and smaller
problem: stale counters from the first call would corrupt it.

This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu


def both(_C, topk_np, E_l, C, rank):
    topk = torch.from_numpy(topk_np).cuda()
    ref = _C.schedule(topk, E_l, C, rank)
    outs = (torch.empty(C, dtype=torch.int32, device="cuda"), torch.empty(C, dtype=torch.int32, device="cuda"),
            torch.empty(1, dtype=torch.int32, device="cuda"), torch.empty(E_l, dtype=torch.int32, device="cuda"))
    _C.schedule_noalloc(topk, E_l, C, rank, *outs)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    return ref, outs


def test_noalloc_schedule_matches_schedule_on_two_calls_in_a_row():
    from mok import _C
    cases = [
        (8, 4096, 8, 32, 4, "random", 7),      # 256 experts over 8 ranks
        (2, 512, 2, 4, 2, "empty_expert", 0),  # much smaller, right after: the shared work area is dirty
    ]
    for R, T, K, E_l, factor, pattern, rank in cases:
        topk = G.schedule_topk(R, T, K, E_l, pattern, seed=21)
        ref, got = both(_C, topk, E_l, T * K * factor, min(rank, R - 1))
        for name, a, b in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), ref, got):
            assert torch.equal(a, b), f"{name} differs between mokb_schedule and mokb_schedule_noalloc"
        assert int(got[2].item()) > 0 and int((got[0] >= 0).sum().item()) > 0


@pytest.mark.parametrize("R,T,K,E_l,factor", [(8, 4096, 8, 128, 2), (1, 16384, 8, 1024, 4)], ids=["ep8_1024_experts", "ep1_1024_experts"])
def test_noalloc_schedule_at_its_expert_limit_matches_the_oracle(R, T, K, E_l, factor):
    """At 1024 experts the per-column counters of the usual geometry (2 or 8 row chunks per column) would need 8 or
    32 MiB; the entry point falls back to fewer chunks until they fit its 4 MiB area.  The schedule must not depend
    on that choice: it has to equal the CPU oracle's and mokb_schedule's (which keeps the usual geometry) bit for bit."""
    from mok import _C
    from oracle import mok_oracle as O
    topk = G.schedule_topk(R, T, K, E_l, "random", seed=23)
    rank = R - 1
    C = T * K * factor
    ref, got = both(_C, topk, E_l, C, rank)
    want = O.schedule(topk, E_l, C, rank)
    n = int(want[2][0])
    for name, w, a, b in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), want, ref, got):
        assert torch.equal(a, b), f"{name} differs between mokb_schedule and mokb_schedule_noalloc"
        w, b = torch.from_numpy(np.asarray(w)), b.cpu()
        if name == "peer_token_idx":                    # defined on scheduled rows only (padding rows: -1 here)
            real = torch.from_numpy(np.asarray(want[0])[:n] >= 0)
            assert torch.equal(w[:n][real], b[:n][real]), name
        else:
            assert torch.equal(w.to(b.dtype), b), f"{name} differs from the oracle"


def test_noalloc_schedule_rejects_sizes_beyond_its_limit():
    from mok import _C
    topk = torch.zeros(4, 512, 1, dtype=torch.int32, device="cuda")
    outs = (torch.empty(512, dtype=torch.int32, device="cuda"), torch.empty(512, dtype=torch.int32, device="cuda"),
            torch.empty(1, dtype=torch.int32, device="cuda"), torch.empty(300, dtype=torch.int32, device="cuda"))
    with pytest.raises(_C.MokError, match="limit of 1024 experts"):
        _C.schedule_noalloc(topk, 300, 512, 0, *outs)          # 4 ranks x 300 experts = 1200 > 1024
