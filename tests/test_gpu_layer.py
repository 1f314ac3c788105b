"""GPU parity tests of the whole layer through mok.functional (EP = 1): against the CPU
oracle on every intermediate, and against the golden fixtures produced by the reference's
own PyTorch implementation."""
import os

import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.golden import make_golden as G
from tests.gpu_common import assert_close, init_single_rank_group, to_dev

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

CTX_KEYS = ("x_routed", "gate_shared", "gate_routed", "up_shared", "up_routed", "hidden_shared", "hidden_routed")
GRAD_KEYS = ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
             "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def run_layer(inp_cpu, E_l, *, limit=None, MB=None, mb=256, recompute=False, mult=0.5):
    import mok
    from mok import _C, functional as F
    group = init_single_rank_group()
    inp = to_dev(inp_cpu)
    T, H = inp.x.shape
    K = inp.top_experts.shape[1]
    cfg = F.MoKConfig(minibatch_size=mb, macrobatch_size=MB or T * K * 2, schedule_capacity_multiplier=mult)
    ws = F.get_workspace(cfg, group, device=torch.device("cuda", 0), num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
    out, ctx = F.forward(cfg, ws, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
                         inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down, limit)
    # the backward replays later macrobatches into the context buffers (as the reference does): keep what the forward saved
    import types
    saved = types.SimpleNamespace(**{k: getattr(ctx, k).clone() for k in CTX_KEYS})
    ctx2 = None
    if recompute:
        ctx2 = F.recompute_forward_context(cfg, ws, sched, inp.x, inp.w_shared_gate, inp.w_shared_up,
                                           inp.w_routed_gate, inp.w_routed_up, limit)
    grads = F.backward(cfg, ws, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate,
                       inp.w_shared_up, inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down, limit)
    torch.cuda.synchronize()
    assert _C.check_status() == 0, _C.status_detail()
    return sched, out, saved, ctx2, grads, ws


@pytest.mark.parametrize("shape", [
    dict(T=512, H=256, I=256, E=4, K=2, routing="router", limit=None),
    dict(T=1024, H=1024, I=512, E=8, K=2, routing="router", limit=None),     # config 1 of the benchmark
    dict(T=512, H=512, I=384, E=6, K=3, routing="gaussian", limit=2.0),      # I not a multiple of 256, clamped
    dict(T=512, H=256, I=128, E=16, K=1, routing="zipf", limit=None, mult=9.0, MB=4608),   # mostly padding, top-1
    dict(T=512, H=1280, I=1408, E=8, K=6, routing="gaussian", limit=None),   # config 5's expert width (11 * 128) and top-6
    dict(T=512, H=1024, I=1536, E=16, K=8, routing="zipf", limit=None, mult=1.0),   # config 4: Zipf routing, multiplier 1.0
], ids=["min", "c1", "i384_clamp", "zipf_top1", "c5_width", "c4_zipf"])
def test_layer_bf16_vs_oracle(shape):
    shape = dict(shape)
    limit, mult, MB = shape.pop("limit"), shape.pop("mult", 0.5), shape.pop("MB", None)
    ranks = O.make_inputs(R=1, seed=3, **shape)
    ref = O.layer_forward_backward(ranks, swiglu_limit=limit, schedule_capacity_factor=max(2, int(mult)))[0]
    sched, out, ctx, _, grads, ws = run_layer(ranks[0], shape["E"], limit=limit, mult=mult, MB=MB)
    # schedule: bit exact
    np.testing.assert_array_equal(sched.peer_rank.cpu().numpy(), ref["peer_rank"])
    np.testing.assert_array_equal(sched.peer_token_idx.cpu().numpy(), ref["peer_token_idx"])
    np.testing.assert_array_equal(sched.tokens_per_expert.cpu().numpy(), ref["tokens_per_expert"])
    N = int(ref["num_tokens"][0])
    # dispatch is an exact copy
    assert torch.equal(ctx.x_routed[:N].cpu(), ref["x_routed"])
    tol = O.BF16_TOLERANCE
    tight = (0.13, 4e-3)
    for k in CTX_KEYS[1:]:
        got = getattr(ctx, k)
        r = ref[k]
        assert_close(k, r, got[: r.shape[0]], tight)
    assert_close("combine_buffer", ref["combine_buffer"], ws.combine_buffer, tight)
    assert_close("output", ref["output"], out, tight)
    for k, got in zip(GRAD_KEYS, grads):
        assert_close(k, ref[k], got, tol)
        mx, rel = O.error_stats(ref[k], got.cpu())
        assert rel < 8e-3, (k, rel)


@pytest.mark.parametrize("case", G.LAYER_CASES[:2], ids=lambda c: c[0])
def test_layer_bf16_vs_reference_golden(case):
    golden = np.load(os.path.join(HERE, "golden", "layer_golden.npz"))
    name, R, T, H, I, E, K, routing, limit = case
    ranks = O.make_inputs(R=R, T=T, H=H, I=I, E=E, K=K, seed=5, routing=routing)
    sched, out, ctx, _, grads, ws = run_layer(ranks[0], E, limit=limit)
    got = dict(zip(GRAD_KEYS, grads), output=out)
    for k in G.LAYER_OUT:
        ref = golden[f"layer_{name}_rank0_{k}"]
        ref = torch.from_numpy(ref) if ref.dtype == np.float32 else torch.from_numpy(ref.view(np.int16).copy()).view(torch.bfloat16)
        g = got[k]
        if k.startswith("d_w_routed"):
            g = g[:, ::4]
        assert_close(k, ref, g, O.BF16_TOLERANCE)


def test_recompute_is_bit_identical_and_runs_are_deterministic():
    ranks = O.make_inputs(R=1, T=512, H=512, I=256, E=8, K=4, seed=11, routing="gaussian")
    s1, out1, ctx1, ctx1b, g1, _ = run_layer(ranks[0], 8, recompute=True)
    s2, out2, ctx2, _, g2, _ = run_layer(ranks[0], 8)
    N = int(s1.num_tokens.item())
    for k in CTX_KEYS:
        a, b, c = getattr(ctx1, k), getattr(ctx1b, k), getattr(ctx2, k)
        n = N if a.shape[0] != 512 else 512
        assert torch.equal(a[:n], b[:n]), f"recompute differs from forward on {k}"
        assert torch.equal(a[:n], c[:n]), f"two runs differ on {k}"
    assert torch.equal(out1, out2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("MB,mb", [(512, 256), (768, 256), (1024, 512)])
def test_several_macrobatches_with_replay_match_the_single_macrobatch_result(MB, mb):
    # capacity 2048 rows, ~1300-1500 of them used: 2-3 populated macrobatches and at least one empty one
    ranks = O.make_inputs(R=1, T=512, H=256, I=256, E=4, K=2, seed=3, routing="gaussian")
    ref = O.layer_forward_backward(ranks)[0]
    N = int(ref["num_tokens"][0])
    assert N > MB
    sched, out, ctx, ctx2, grads, ws = run_layer(ranks[0], 4, MB=MB, mb=mb, recompute=True)
    # the saved context is macrobatch 0, and recompute rebuilds exactly that
    assert torch.equal(ctx.x_routed.cpu(), ref["x_routed"][:MB])
    assert_close("gate_routed", ref["gate_routed"][:MB], ctx.gate_routed, (0.13, 4e-3))
    for k in CTX_KEYS:
        assert torch.equal(getattr(ctx, k), getattr(ctx2, k)), k
    assert_close("combine_buffer", ref["combine_buffer"], ws.combine_buffer, (0.13, 4e-3))
    assert_close("output", ref["output"], out, (0.13, 4e-3))
    for k, got in zip(GRAD_KEYS, grads):
        assert_close(k, ref[k], got, O.BF16_TOLERANCE)
        assert O.error_stats(ref[k], got.cpu())[1] < 8e-3, k
    # bit-reproducible across runs as well
    _, out_b, _, _, grads_b, _ = run_layer(ranks[0], 4, MB=MB, mb=mb)
    assert torch.equal(out, out_b) and all(torch.equal(a, b) for a, b in zip(grads, grads_b))


def test_launch_timeline_records_every_phase_in_order():
    from mok import _C
    ranks = O.make_inputs(R=1, T=512, H=256, I=256, E=4, K=2, seed=3, routing="gaussian")
    run_layer(ranks[0], 4)                   # warm-up: streams, events, function attributes
    torch.cuda.synchronize()
    _C.trace_begin()
    run_layer(ranks[0], 4)
    recs = _C.trace_end()
    tags = [r[0] for r in recs]
    for expected in ("schedule", "dispatch", "gemm_bf16_gate_up_swiglu", "gemm_bf16_nt", "gemm_bf16_fwd_routed",
                     "fwd_epilogue", "dispatch_scaled", "gemm_bf16_nn", "swiglu_bwd", "gemm_bf16_wgrad", "bwd_epilogue"):
        assert expected in tags, expected
    assert "combine" not in tags             # the rows go home from the epilogues of the GEMMs that compute them
    assert tags.count("gemm_bf16_fwd_routed") == 1      # one persistent launch for every window of the routed forward
    assert all(0.0 <= b <= e for _, _, _, b, e in recs)
    assert len({r[2] for r in recs}) == 2    # the caller's stream and the side stream of the pulls
    first = {t: min(r[3] for r in recs if r[0] == t) for t in set(tags)}
    assert (first["schedule"] < first["dispatch"] < first["gemm_bf16_fwd_routed"] < first["fwd_epilogue"]
            < first["dispatch_scaled"] < first["bwd_epilogue"])
    assert _C.trace_end() == []              # recording has stopped


def test_inputs_already_in_the_workspace_buffers_skip_the_staging_copies_and_change_nothing():
    from mok import _C, functional as F
    ranks = O.make_inputs(R=1, T=512, H=256, I=256, E=4, K=2, seed=9, routing="gaussian")
    _, out_ref, _, _, grads_ref, _ = run_layer(ranks[0], 4)
    group = init_single_rank_group()
    inp = to_dev(ranks[0])
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=2048)
    ws = F.get_workspace(cfg, group, device=torch.device("cuda", 0), num_local_tokens=512, hidden_size=256, topk=2)
    ws.x_buffer.copy_(inp.x)
    ws.router_weight_buffer.copy_(inp.router_weights)
    ws.d_y_buffer.copy_(inp.grad_output)
    sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=4)
    w = (inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down)
    out, ctx = F.forward(cfg, ws, sched, ws.x_buffer, ws.router_weight_buffer, *w)
    grads = F.backward(cfg, ws, sched, ctx, ws.d_y_buffer, ws.x_buffer, ws.router_weight_buffer, *w)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    assert torch.equal(out, out_ref) and all(torch.equal(a, b) for a, b in zip(grads, grads_ref))


@pytest.mark.parametrize("mxfp8", [False, True], ids=["bf16", "mxfp8"])
def test_a_corrupted_schedule_sets_a_status_code_instead_of_reaching_outside_the_buffers(mxfp8):
    """One schedule entry rewritten to a route index far outside [0, tokens * topk): forward and backward run to the
    end, the row is treated as padding, and the status words say MOKB_ST_BAD_INDEX with the row and the index."""
    from mok import _C, ops, functional as F
    group = init_single_rank_group()
    E_l, T, H, I, K = 4, 512, 256, 256, 2
    inp = to_dev(O.make_inputs(R=1, T=T, H=H, I=I, E=E_l, K=K, seed=21, routing="gaussian")[0])
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=T * K * 2)
    ws = F.get_workspace(cfg, group, device=torch.device("cuda", 0), num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
    live = torch.nonzero(sched.peer_rank[: int(sched.num_tokens.item())] >= 0).flatten()
    bad_row, bad_idx = int(live[live.numel() // 3]), 1 << 27
    sched.peer_token_idx[bad_row] = bad_idx
    if mxfp8:
        q = [ops.mxfp8_quantize(w, True, True) for w in (inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down)]
        fw = [(a, b) for a, b, _, _ in q]
        bw = [q[0], q[1], (q[2][2], q[2][3])]
    else:
        fw = bw = [inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down]
    out, ctx = F.forward(cfg, ws, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down, *fw)
    torch.cuda.synchronize()
    assert _C.check_status() == _C.ST_BAD_INDEX
    assert _C.status_detail()[2:] == [bad_row, bad_idx]
    assert torch.isfinite(out.float()).all()
    F.backward(cfg, ws, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
               inp.w_shared_down, *bw)
    torch.cuda.synchronize()
    assert _C.check_status() == _C.ST_BAD_INDEX
    assert _C.status_detail()[2:] == [bad_row, bad_idx]
