"""GPU parity of the MXFP8 layer (routed experts in block-scaled E4M3) through mok.functional at EP = 1:
against the CPU oracle's MXFP8 dataflow (tight) and against the BF16 result under the reference's
MXFP8 tolerance (max abs <= 1.0, relative <= 0.1; tests/utils.py:8 of the reference)."""
import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.gpu_common import assert_close, init_single_rank_group, to_dev

pytestmark = pytest.mark.gpu

GRAD_KEYS = ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
             "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def run_mxfp8(inp_cpu, E_l, *, limit=None, recompute=False, MB=None, mb=256, mult=0.5):
    from mok import _C, functional as F, ops
    group = init_single_rank_group()
    inp = to_dev(inp_cpu)
    T, H = inp.x.shape
    K = inp.top_experts.shape[1]
    cfg = F.MoKConfig(minibatch_size=mb, macrobatch_size=MB or T * K * 2, schedule_capacity_multiplier=mult)
    ws = F.get_workspace(cfg, group, device=torch.device("cuda", 0), num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
    gq, gs, gtq, gts = ops.mxfp8_quantize(inp.w_routed_gate, True, True)
    uq, us, utq, uts = ops.mxfp8_quantize(inp.w_routed_up, True, True)
    dq, ds, dtq, dts = ops.mxfp8_quantize(inp.w_routed_down, True, True)
    out, ctx = F.forward(cfg, ws, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down,
                         (gq, gs), (uq, us), (dq, ds), limit)
    ctx2 = None
    if recompute:
        ctx2 = F.recompute_forward_context(cfg, ws, sched, inp.x, inp.w_shared_gate, inp.w_shared_up, (gq, gs), (uq, us), limit)
    grads = F.backward(cfg, ws, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
                       inp.w_shared_down, (gq, gs, gtq, gts), (uq, us, utq, uts), (dtq, dts), limit)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    return sched, out, ctx, ctx2, grads, ws


@pytest.mark.parametrize("shape", [
    dict(T=512, H=256, I=256, E=4, K=2, routing="router", limit=None),
    dict(T=1024, H=1024, I=512, E=8, K=2, routing="router", limit=None),      # config 3 of the benchmark (MXFP8 of config 1)
    dict(T=512, H=512, I=384, E=6, K=3, routing="gaussian", limit=2.0),
    dict(T=512, H=1280, I=1408, E=8, K=6, routing="gaussian", limit=None),   # config 5's expert width (11 * 128) and top-6
    dict(T=512, H=1024, I=1536, E=16, K=8, routing="zipf", limit=None, mult=1.0),   # config 4: Zipf routing, multiplier 1.0
], ids=["min", "c3", "i384_clamp", "c5_width", "c4_zipf"])
def test_layer_mxfp8_vs_oracle(shape):
    shape = dict(shape)
    limit, mult = shape.pop("limit"), shape.pop("mult", 0.5)
    ranks = O.make_inputs(R=1, seed=3, **shape)
    # the reference's tolerance is absolute; use its gradient scale (d_output ~ N(0,1) * H^-0.5, tests/utils.py:93)
    ranks[0].grad_output = (ranks[0].grad_output.float() * shape["H"] ** -0.5).to(torch.bfloat16)
    ref = O.layer_forward_backward(ranks, swiglu_limit=limit, mxfp8=True)[0]
    ref_bf16 = O.layer_forward_backward(ranks, swiglu_limit=limit)[0]
    sched, out, ctx, _, grads, ws = run_mxfp8(ranks[0], shape["E"], limit=limit, mult=mult)
    N = int(ref["num_tokens"][0])
    # x_routed^T quantised along tokens: exact copy + byte-exact codec
    xq, xs, _, _ = O.mxfp8_quantize(ref["x_routed"].T.contiguous(), True, False)
    assert torch.equal(ctx.x_routed[0][:, :N].cpu().view(torch.uint8), xq.view(torch.uint8))
    assert torch.equal(O.unpack_scales(ctx.x_routed[1].cpu())[:, : N // 32], O.unpack_scales(xs))
    # saved gate/up: de-quantised values close to the oracle's bf16 gate/up
    g = O.dequantize(ctx.gate_routed[0][:N].cpu(), ctx.gate_routed[1][: N // 128].cpu())
    assert_close("gate", ref["gate_routed"], g, (0.5, 0.05))
    tight = (0.25, 0.02)
    assert_close("output vs mxfp8 oracle", ref["output"], out, tight)
    for k, got in zip(GRAD_KEYS, grads):
        assert_close(k + " vs mxfp8 oracle", ref[k], got, (0.25, 0.03))
        assert_close(k + " vs bf16", ref_bf16[k], got, O.MXFP8_TOLERANCE)
    assert_close("output vs bf16", ref_bf16["output"], out, O.MXFP8_TOLERANCE)
    # the shared expert stays BF16: its gradients are those of the BF16 path
    assert_close("d_w_shared_down", ref_bf16["d_w_shared_down"], grads[7], O.BF16_TOLERANCE)


def test_mxfp8_recompute_is_bit_identical_and_deterministic():
    ranks = O.make_inputs(R=1, T=512, H=512, I=256, E=8, K=4, seed=11, routing="gaussian")
    s1, out1, ctx1, ctx1b, g1, _ = run_mxfp8(ranks[0], 8, recompute=True)
    s2, out2, ctx2, _, g2, _ = run_mxfp8(ranks[0], 8)
    N = int(s1.num_tokens.item())

    def live(t, transposed):
        # only rows (columns, for the token-axis tensors) below num_tokens are defined
        t = t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t
        if t.ndim == 4:
            return t[:, : N // 128] if transposed else t[: N // 128]
        return t[:, :N] if transposed else t[:N]
    for name, tr in (("x_routed", True), ("gate_routed", False), ("up_routed", False), ("hidden_routed", True)):
        for a, b, c in zip(getattr(ctx1, name), getattr(ctx1b, name), getattr(ctx2, name)):
            assert torch.equal(live(a, tr), live(b, tr)), f"recompute differs on {name}"
            assert torch.equal(live(a, tr), live(c, tr)), f"two runs differ on {name}"
    for name in ("gate_shared", "up_shared", "hidden_shared"):
        assert torch.equal(getattr(ctx1, name), getattr(ctx1b, name))
    assert torch.equal(out1, out2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("MB,mb", [(512, 256), (768, 256), (1024, 512)])
def test_mxfp8_several_macrobatches_with_replay_match_the_single_macrobatch_result(MB, mb):
    # capacity 2048 rows, ~1300-1500 of them used: 2-3 populated macrobatches and at least one empty one.
    # Macrobatch boundaries are multiples of 256 rows, so no 32-token scale block straddles one: everything
    # except the accumulation order of the routed weight gradients is the same arithmetic as in one macrobatch.
    ranks = O.make_inputs(R=1, T=512, H=256, I=256, E=4, K=2, seed=3, routing="gaussian")
    ranks[0].grad_output = (ranks[0].grad_output.float() * 256 ** -0.5).to(torch.bfloat16)
    s1, out1, ctx1, _, g1, ws1 = run_mxfp8(ranks[0], 4)
    N = int(s1.num_tokens.item())
    assert N > MB
    combine1 = ws1.combine_buffer.clone()
    sm, outm, ctxm, ctxm2, gm, wsm = run_mxfp8(ranks[0], 4, MB=MB, mb=mb, recompute=True)
    assert torch.equal(out1, outm)
    assert torch.equal(combine1, wsm.combine_buffer)
    named = dict(zip(GRAD_KEYS, zip(g1, gm)))
    for k in ("d_x", "d_router_weights", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down"):
        assert torch.equal(*named[k]), k
    for k in ("d_w_routed_gate", "d_w_routed_up", "d_w_routed_down"):       # bf16 accumulation across macrobatches
        a, b = named[k]
        assert_close(k, a.cpu(), b, (0.02, 8e-3))
    # recompute rebuilds macrobatch 0, which is what the forward saved (the backward has since replayed later ones)
    for pair_single, pair_re, transposed in ((ctx1.x_routed, ctxm2.x_routed, True), (ctx1.gate_routed, ctxm2.gate_routed, False),
                                             (ctx1.up_routed, ctxm2.up_routed, False), (ctx1.hidden_routed, ctxm2.hidden_routed, True)):
        a, b = pair_single[0].view(torch.uint8), pair_re[0].view(torch.uint8)
        if transposed:
            assert torch.equal(a[:, :MB], b[:, :MB])
        else:
            assert torch.equal(a[:MB], b[:MB])
    # bit-reproducible across runs
    _, outb, _, _, gb, _ = run_mxfp8(ranks[0], 4, MB=MB, mb=mb)
    assert torch.equal(outm, outb) and all(torch.equal(a, b) for a, b in zip(gm, gb))
