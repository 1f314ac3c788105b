"""The CPU oracle against fixtures produced by the reference's own PyTorch
implementation (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.golden import make_golden as G

HERE = os.path.dirname(os.path.abspath(__file__))
OPS = np.load(os.path.join(HERE, "golden", "ops_golden.npz"))
LAYER = np.load(os.path.join(HERE, "golden", "layer_golden.npz"))


def bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.parametrize("case", G.SCHEDULE_CASES, ids=lambda c: c[0])
def test_schedule_matches_reference(case):
    name, R, T, K, E_l, factor, pattern = case
    topk = G.schedule_topk(R, T, K, E_l, pattern)
    for rank in sorted({0, R - 1}):
        pr, pt, nt, tpe = O.schedule(topk, E_l, T * K * factor, rank)
        key = f"sched_{name}_rank{rank}"
        np.testing.assert_array_equal(pr, OPS[key + "_peer_rank"])
        np.testing.assert_array_equal(pt, OPS[key + "_peer_token_idx"])
        np.testing.assert_array_equal(nt, OPS[key + "_num_tokens"])
        np.testing.assert_array_equal(tpe, OPS[key + "_tokens_per_expert"])


def test_schedule_bruteforce_agrees():
    topk = G.schedule_topk(2, 512, 2, 2, "random", seed=5)[:, :128]
    a = O.schedule(topk, 2, 1024, 1)
    b = O.schedule_bruteforce(topk, 2, 1024, 1)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)


def test_schedule_overflow_is_an_error():
    topk = np.zeros((4, 512, 1), np.int32)      # every route to expert 0
    with pytest.raises(ValueError):
        O.schedule(topk, 1, 512, 0)


@pytest.mark.parametrize("name", ["q2d", "q3d", "qwide"])
def test_quantiser_bytes_match_reference(name):
    x = bf16(OPS[name + "_in"])
    q, s, qt, st = O.mxfp8_quantize(x, True, True)
    np.testing.assert_array_equal(q.view(torch.uint8).numpy(), OPS[name + "_fp8"])
    np.testing.assert_array_equal(s.numpy(), OPS[name + "_sc"])
    np.testing.assert_array_equal(qt.view(torch.uint8).numpy(), OPS[name + "_fp8_t"])
    np.testing.assert_array_equal(st.numpy(), OPS[name + "_sc_t"])


def test_quantiser_zero_block_and_roundtrip():
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    x[0, :32] = 448.0
    x[1, :32] = 1.75 * 2.0 ** -20
    q, s, _, _ = O.mxfp8_quantize(x, True, False)
    sc = O.unpack_scales(s)
    assert sc[0, 0] == 127 and sc[1, 0] == 127 - 28 and sc[2, 0] == 88   # all-zero block: 2^-39
    d = O.dequantize(q, s)
    assert torch.equal(d[0, :32], x[0, :32].float()) and torch.equal(d[2], torch.zeros(128))
    assert torch.equal(O.unpack_scales(O.pack_scales(sc)), sc)


def test_swiglu_and_epilogues_match_reference():
    gate, up = bf16(OPS["swiglu_gate"]), bf16(OPS["swiglu_up"])
    for key, lim in (("swiglu_none", None), ("swiglu_clamp4", 4.0)):
        ref = bf16(OPS[key])
        got = O.swiglu_fwd(gate, up, lim)
        # the reference's unclamped branch multiplies two bf16 tensors (tests/utils.py:230),
        # i.e. rounds silu(g) before the product; one bf16 ulp of slack covers that
        mx, rel = O.error_stats(ref, got)
        assert rel < 4e-3, (key, mx, rel)
    y, comb, w = bf16(OPS["epi_y"]), bf16(OPS["epi_comb"]), torch.from_numpy(OPS["epi_w"])
    mx, rel = O.error_stats(bf16(OPS["epi_fwd"]), O.fwd_epilogue(y, comb, w))
    assert rel < 2e-3
    mx, rel = O.error_stats(bf16(OPS["epi_bwd"]), O.bwd_epilogue(y, comb))
    assert rel < 2e-3


def test_swiglu_backward_is_the_derivative():
    g = torch.randn(32, 64, dtype=torch.float64, requires_grad=True)
    u = torch.randn(32, 64, dtype=torch.float64, requires_grad=True)
    dh = torch.randn(32, 64, dtype=torch.float64)
    (torch.nn.functional.silu(g) * u).backward(dh)
    dg, du, hid = O.swiglu_bwd(g.detach().float(), u.detach().float(), dh.float(), None)
    assert O.error_stats(g.grad, dg)[1] < 5e-3 and O.error_stats(u.grad, du)[1] < 5e-3


@pytest.mark.parametrize("case", G.LAYER_CASES, ids=lambda c: c[0])
def test_layer_bf16_matches_reference(case):
    name, R, T, H, I, E, K, routing, limit = case
    ranks = O.make_inputs(R=R, T=T, H=H, I=I, E=E, K=K, seed=5, routing=routing)
    outs = O.layer_forward_backward(ranks, swiglu_limit=limit)
    for r in range(R):
        chk = LAYER[f"layer_{name}_rank{r}_input_checksum"]
        inp = ranks[r]
        mine = [G.checksum(inp.x), G.checksum(inp.top_experts), G.checksum(inp.w_routed_gate), G.checksum(inp.grad_output)]
        assert list(chk) == mine, "seeded inputs differ from the ones the fixture was generated with"
        for k in G.LAYER_OUT:
            ref = LAYER[f"layer_{name}_rank{r}_{k}"]
            ref = torch.from_numpy(ref) if ref.dtype == np.float32 else bf16(ref)
            got = outs[r][k]
            if k.startswith("d_w_routed"):
                got = got[:, ::4]
            mx, rel = O.error_stats(ref, got)
            assert mx <= O.BF16_TOLERANCE[0] and rel <= O.BF16_TOLERANCE[1], (k, r, mx, rel)


def test_layer_mxfp8_within_reference_tolerance_of_bf16():
    ranks = O.make_inputs(R=1, T=512, H=256, I=256, E=4, K=2, seed=5, routing="router")
    a = O.layer_forward_backward(ranks)[0]
    b = O.layer_forward_backward(ranks, mxfp8=True)[0]
    for k in G.LAYER_OUT:
        mx, rel = O.error_stats(a[k], b[k])
        assert mx <= O.MXFP8_TOLERANCE[0] and rel <= O.MXFP8_TOLERANCE[1], (k, mx, rel)
        # the shared expert stays BF16 in MXFP8 mode; routed results must really differ
        assert (rel == 0) == k.startswith("d_w_shared"), (k, rel)
