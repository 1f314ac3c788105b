"""The operator surface under torch.compile: one graph for build_schedule + forward + backward with the `mok::`
operators in the reference's order (tests/test_misc.py:1262-1521 of the reference, which traces under FakeTensorMode
with a capture backend), the mutation schemas it pins (tests/test_misc.py:1218-1259), and torch.library.opcheck on
operators with real tensors."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_custom_op_mutation_schemas():
    from mok import ops, ops_mxfp8  # noqa: F401
    expected = {
        "all_gather_top_experts": {"all_gather_top_experts_buffer"},
        "barrier_all": {"barrier_buffer", "target"},
        "schedule": set(),
        "mxfp8_quantize": set(),
        "dispatch_mlp_swiglu_combine_fwd_mxfp8": {"combine_buffer"},
        "dispatch_mlp_swiglu_combine_fwd_bf16": {"combine_buffer"},
        "recompute_forward_context_mxfp8": set(),
        "recompute_forward_context_bf16": set(),
        "dispatch_mlp_swiglu_combine_bwd_mxfp8": {"d_x_routed_buffer", "d_router_weight_buffer", "x_fp8_t_routed", "x_sc_t_routed",
                                                  "gate_fp8_routed", "gate_sc_routed", "up_fp8_routed", "up_sc_routed",
                                                  "hidden_fp8_t_routed", "hidden_sc_t_routed"},
        "dispatch_mlp_swiglu_combine_bwd_bf16": {"d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed",
                                                 "up_routed", "hidden_routed"},
        "fwd_epilogue": set(),
        "bwd_epilogue": set(),
    }
    actual = {}
    for name in expected:
        schema = getattr(torch.ops.mok, name).default._schema
        actual[name] = {a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write}
    assert actual == expected


def fake_workspace(F, device, T, H, K, capacity):
    def t(shape, dtype):
        return torch.empty(shape, device=device, dtype=dtype)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    return F.MoKWorkspace(
        group_name="fake", ep_rank=0, ep_size=1, device=device, num_local_tokens=T, hidden_size=H, topk=K,
        schedule_capacity=capacity,
        x_buffer=t((T, H), bf), x_buffer_handle=None, x_buffer_ptrs=[16],
        combine_buffer=t((T * K, H), bf), combine_buffer_handle=None, combine_buffer_ptrs=[16],
        d_y_buffer=t((T, H), bf), d_y_buffer_handle=None, d_y_buffer_ptrs=[16],
        d_x_routed_buffer=t((T * K, H), bf), d_x_routed_buffer_handle=None, d_x_routed_buffer_ptrs=[16],
        router_weight_buffer=t((T, K), f32), router_weight_buffer_handle=None, router_weight_buffer_ptrs=[16],
        d_router_weight_buffer=t((T, K), f32), d_router_weight_buffer_handle=None, d_router_weight_buffer_ptrs=[16],
        all_gather_top_experts_buffer=t((1, T, K), i32), all_gather_top_experts_buffer_handle=None,
        all_gather_top_experts_buffer_multicast_ptr=16,
        barrier_buffer=t((1,), i32), barrier_buffer_handle=None, barrier_buffer_ptrs=[16], barrier_buffer_multicast_ptr=16,
        barrier_target=t((1,), i32), all_gather_top_experts_buffer_ptrs=[16])


@pytest.mark.parametrize("precision", ["bf16", "mxfp8"])
def test_compile_fullgraph_captures_the_operators_in_order(precision):
    from torch._subclasses.fake_tensor import FakeTensorMode
    from mok import functional as F, ops
    T, H, I, E_l, K = 512, 1024, 256, 4, 2
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=512)
    captured = []

    def capture_backend(gm, _inputs):
        captured.append(gm)
        return gm.forward

    with FakeTensorMode():
        device = torch.device("cuda", torch.cuda.current_device())
        ws = fake_workspace(F, device, T, H, K, 4096)

        def t(shape, dtype=torch.bfloat16):
            return torch.empty(shape, device=device, dtype=dtype)
        x, gy = t((T, H)), t((T, H))
        te, rw = t((T, K), torch.int64), t((T, K), torch.float32)
        sg, su, sd = t((I, H)), t((I, H)), t((H, I))
        rg, ru, rd = t((E_l, I, H)), t((E_l, I, H)), t((E_l, H, I))

        def complete_path(x, te, rw, gy, sg, su, sd, rg, ru, rd):
            sched = F.build_schedule(ws, cfg, te, num_local_experts=E_l)
            if precision == "mxfp8":
                qg, qu, qd = (ops.mxfp8_quantize(w, True, True) for w in (rg, ru, rd))
                fwd_w = ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
                bwd_w = (qg, qu, (qd[2], qd[3]))
            else:
                fwd_w = bwd_w = (rg, ru, rd)
            out, ctx = F.forward(cfg, ws, sched, x, rw, sg, su, sd, *fwd_w)
            grads = F.backward(cfg, ws, sched, ctx, gy, x, rw, sg, su, sd, *bwd_w)
            return (out, *grads)

        torch._dynamo.reset()
        compiled = torch.compile(complete_path, backend=capture_backend, fullgraph=True)
        outs = compiled(x, te, rw, gy, sg, su, sd, rg, ru, rd)
        again = compiled(x, te, rw, gy, sg, su, sd, rg, ru, rd)
        want = [((T, H), torch.bfloat16), ((T, H), torch.bfloat16), ((T, K), torch.float32),
                ((E_l, I, H), torch.bfloat16), ((E_l, I, H), torch.bfloat16), ((E_l, H, I), torch.bfloat16),
                ((I, H), torch.bfloat16), ((I, H), torch.bfloat16), ((H, I), torch.bfloat16)]
        for got in (outs, again):
            assert [(tuple(o.shape), o.dtype) for o in got] == want
    assert len(captured) == 1
    targets = [str(n.target) for n in captured[0].graph.nodes if n.op == "call_function" and "mok" in str(n.target)]
    expected = ["mok.all_gather_top_experts.default", "mok.barrier_all.default", "mok.schedule.default",
                "mok.barrier_all.default", f"mok.dispatch_mlp_swiglu_combine_fwd_{precision}.default",
                "mok.barrier_all.default", "mok.fwd_epilogue.default",
                "mok.barrier_all.default", f"mok.dispatch_mlp_swiglu_combine_bwd_{precision}.default",
                "mok.barrier_all.default", "mok.bwd_epilogue.default"]
    if precision == "mxfp8":
        expected = expected[:3] + ["mok.mxfp8_quantize.default"] * 3 + expected[3:]
    assert targets == expected


def test_opcheck_on_operators_with_real_tensors():
    from mok import ops
    opcheck = torch.library.opcheck
    tests = ("test_schema", "test_faketensor")
    topk = torch.randint(0, 8, (1, 512, 2), dtype=torch.int32, device="cuda")
    opcheck(torch.ops.mok.schedule.default, (topk, 8, 2048, 0), test_utils=tests)
    x = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    opcheck(torch.ops.mok.mxfp8_quantize.default, (x, True, True), test_utils=tests)
    comb = torch.randn(1024, 256, device="cuda").to(torch.bfloat16)
    w = torch.rand(512, 2, device="cuda")
    opcheck(torch.ops.mok.fwd_epilogue.default, (x, comb, w), test_utils=tests)
    opcheck(torch.ops.mok.bwd_epilogue.default, (x, comb), test_utils=tests)
    # a mutating operator: the route gather writes its buffer argument
    buf = torch.zeros(1, 512, 2, dtype=torch.int32, device="cuda")
    opcheck(torch.ops.mok.all_gather_top_experts.default, (topk[0].contiguous(), buf, 0, 0, 2048, [buf.data_ptr()]), test_utils=tests)
