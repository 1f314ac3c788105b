"""Host-side logic that needs no GPU: configuration checks, operator argument validation,
the shape agreement collective over gloo with two ranks, and the multi-rank oracle."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mok_oracle as O


def test_config_validation_matches_reference_rules():
    from mok.functional import MoKConfig, validate_config, schedule_capacity_factor
    ok = MoKConfig()
    validate_config(ok, 148, 16384 * 8 * 4)
    bad = [
        (MoKConfig(fwd_num_comm_sms=3), "even"), (MoKConfig(bwd_num_comm_sms=0), "positive"),
        (MoKConfig(fwd_num_comm_sms=148), "compute SM"), (MoKConfig(minibatch_size=100), "256"),
        (MoKConfig(macrobatch_size=4096 * 3 + 256), "multiple of minibatch"),
        (MoKConfig(all_gather_top_experts_chunk_bytes=24), "multiple of 16"),
        (MoKConfig(all_gather_top_experts_chunk_bytes=4096 * 1024), "capacity"),
        (MoKConfig(all_gather_top_experts_chunk_bytes=2048 * 3), "divide"),
    ]
    for cfg, msg in bad:
        with pytest.raises(ValueError, match=msg):
            validate_config(cfg, 148, 16384 * 8 * 4)
    with pytest.raises(TypeError):
        validate_config(object(), 148, 4096)
    assert schedule_capacity_factor(MoKConfig(), 8) == 4          # 16384*8*4 = 524288 rows at config 2
    assert schedule_capacity_factor(MoKConfig(schedule_capacity_multiplier=1.0), 8) == 8
    assert schedule_capacity_factor(MoKConfig(), 1) == 2


def test_shape_validation():
    from mok.functional import validate_shape_args
    validate_shape_args(512, 256, 1)
    for args in ((256, 256, 1), (600, 256, 1), (512, 100, 1), (512, 256, 0), (512, 256, 256), (512.0, 256, 1)):
        with pytest.raises(ValueError):
            validate_shape_args(*args)


def test_ops_reject_bad_arguments_before_touching_a_device():
    from mok import ops
    t = torch.zeros(1, 512, 2, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA"):
        ops.schedule(t, 4, 2048, 0)
    x = torch.zeros(512, 256, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible by 128"):
        ops.mxfp8_quantize(torch.zeros(100, 128, dtype=torch.bfloat16), True, False)
    with pytest.raises(ValueError, match="at least one"):
        ops.mxfp8_quantize(torch.zeros(128, 128, dtype=torch.bfloat16), False, False)
    with pytest.raises(ValueError, match="topk_weights"):
        ops.fwd_epilogue(x, torch.zeros(1024, 256, dtype=torch.bfloat16), torch.zeros(100, 2))
    with pytest.raises(ValueError, match="d_x_routed_buffer"):
        ops.bwd_epilogue(x, torch.zeros(1000, 256, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="list of positive integers"):
        ops._check_ptrs("barrier_buffer_ptrs", [0, 16])
    with pytest.raises(ValueError, match="match x_ptrs"):
        ops._check_ptrs("combine_buffer_ptrs", [16, 32], 4)
    with pytest.raises(ValueError, match="multiple of minibatch"):
        ops._check_knobs(2, None, 2, 1000, 256)
    with pytest.raises(ValueError, match="swiglu_limit"):
        ops._check_knobs(2, -1.0, 2, 1024, 256)


def test_fake_tensor_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    from mok import ops
    with FakeTensorMode():
        topk = torch.empty(2, 512, 4, dtype=torch.int32, device="cuda")
        pr, pt, nt, tpe = torch.ops.mok.schedule(topk, 8, 8192, 0)
        assert pr.shape == (8192,) and tpe.shape == (8,) and nt.dtype == torch.int32
        x = torch.empty(512, 256, dtype=torch.bfloat16, device="cuda")
        q, s, qt, st = torch.ops.mok.mxfp8_quantize(x, True, False)
        assert q.dtype == torch.float8_e4m3fn and s.shape == (4, 2, 32, 16) and qt is None


def _two_rank_worker(rank, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    from mok.functional import check_identical_shapes
    check_identical_shapes(dist.group.WORLD, torch.device("cpu"), 512, 256, 2)
    try:
        check_identical_shapes(dist.group.WORLD, torch.device("cpu"), 512 + 256 * rank, 256, 2)
        mismatch = False
    except ValueError:
        mismatch = True
    # every rank builds its own schedule from the gathered routes; together they cover each route once
    routes = torch.topk(torch.randn(512, 8, generator=torch.Generator().manual_seed(rank)), 2).indices.to(torch.int32)
    gathered = [torch.empty_like(routes) for _ in range(2)]
    dist.all_gather(gathered, routes)
    topk_all = torch.stack(gathered).numpy()
    pr, pt, nt, tpe = O.schedule(topk_all, 4, 2048, rank)
    n = int(nt[0])
    real = pr[:n] >= 0
    keys = torch.from_numpy(pr[:n][real].astype(np.int64) * 1024 + pt[:n][real])
    all_keys = [torch.empty(2048, dtype=torch.int64) for _ in range(2)]
    padded = torch.full((2048,), -1, dtype=torch.int64)
    padded[: keys.numel()] = keys
    dist.all_gather(all_keys, padded)
    union = torch.cat(all_keys)
    union = union[union >= 0]
    ret[rank] = (mismatch, int(union.numel()), int(union.unique().numel()))
    dist.destroy_process_group()


def test_two_ranks_over_gloo():
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_two_rank_worker, args=(29711, ret), nprocs=2, join=True)
        for r in range(2):
            mismatch, total, unique = ret[r]
            assert mismatch and total == 2 * 512 * 2 and unique == total


def test_oracle_multi_rank_layer_is_consistent_with_single_rank_math():
    # with R ranks, every token's output must equal what a 1-rank layer holding all experts computes
    R, T, H, I, E, K = 2, 512, 256, 128, 4, 2
    ranks = O.make_inputs(R=R, T=T, H=H, I=I, E=E, K=K, seed=1, routing="gaussian")
    outs = O.layer_forward_backward(ranks, with_backward=False)
    allW = [torch.cat([r.w_routed_gate for r in ranks]), torch.cat([r.w_routed_up for r in ranks]),
            torch.cat([r.w_routed_down for r in ranks])]
    for r in range(R):
        one = O.RankInputs(**{**ranks[r].__dict__, "w_routed_gate": allW[0], "w_routed_up": allW[1], "w_routed_down": allW[2]})
        single = O.layer_forward_backward([one], with_backward=False)[0]
        assert torch.equal(single["output"], outs[r]["output"])


def test_whole_layer_traces_under_fake_tensors():
    """Every operator of forward + backward (BF16 and MXFP8) has a meta kernel with the reference's output
    shapes, so the layer can be traced without a device (what torch.compile(fullgraph=True) needs)."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from mok import ops  # noqa: F401
    T, H, I, E_l, K, MB, C = 512, 256, 384, 4, 2, 1024, 2048
    with FakeTensorMode():
        dev = "cuda"
        bf = dict(dtype=torch.bfloat16, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        x = torch.empty(T, H, **bf)
        comb = torch.empty(T * K, H, **bf)
        wsg, wsu, wsd = torch.empty(I, H, **bf), torch.empty(I, H, **bf), torch.empty(H, I, **bf)
        wrg, wru, wrd = torch.empty(E_l, I, H, **bf), torch.empty(E_l, I, H, **bf), torch.empty(E_l, H, I, **bf)
        sched = (torch.empty(C, **i32), torch.empty(C, **i32), torch.empty(1, **i32), torch.empty(E_l, **i32))
        f = torch.ops.mok.dispatch_mlp_swiglu_combine_fwd_bf16(x, [16], comb, [16], wsg, wrg, wsu, wru, wsd, wrd, *sched,
                                                              K, None, 40, MB, 256)
        assert [tuple(t.shape) for t in f] == [(MB, H), (T, I), (MB, I), (T, I), (MB, I), (T, I), (MB, I), (T, H), (MB, H)]
        rw = torch.empty(T, K, device=dev)
        b = torch.ops.mok.dispatch_mlp_swiglu_combine_bwd_bf16(x, [16], comb, [16], rw, [16], rw, [16], wsg, wrg, wsu, wru,
                                                              wsd, wrd, f[0], f[1], f[2], f[3], f[4], f[5], f[6], x, [16],
                                                              *sched, K, None, 28, MB, 256)
        assert len(b) == 15 and tuple(b[10].shape) == (E_l, I, H) and tuple(b[14].shape) == (E_l, H, I)
        assert tuple(torch.ops.mok.fwd_epilogue(f[7], comb, rw).shape) == (T, H)
        assert tuple(torch.ops.mok.bwd_epilogue(b[0], comb).shape) == (T, H)
        # MXFP8
        q = lambda t: torch.ops.mok.mxfp8_quantize(t, True, True)
        gq, uq, dq = q(wrg), q(wru), q(wrd)
        assert tuple(gq[2].shape) == (E_l, H, I) and tuple(gq[3].shape) == (E_l * H // 128, I // 128, 32, 16)
        fm = torch.ops.mok.dispatch_mlp_swiglu_combine_fwd_mxfp8(x, [16], comb, [16], wsg, gq[0], gq[1], wsu, uq[0], uq[1],
                                                                wsd, dq[0], dq[1], *sched, K, None, 40, MB, 256)
        assert len(fm) == 13 and tuple(fm[0].shape) == (H, MB) and fm[0].dtype == torch.float8_e4m3fn
        assert tuple(fm[10].shape) == (I // 128, MB // 128, 32, 16) and tuple(fm[12].shape) == (MB, H)
        rm = torch.ops.mok.recompute_forward_context_mxfp8(x, [16], wsg, gq[0], gq[1], wsu, uq[0], uq[1], *sched, K, None,
                                                          40, MB, 256)
        assert len(rm) == 11
        bm = torch.ops.mok.dispatch_mlp_swiglu_combine_bwd_mxfp8(
            x, [16], comb, [16], rw, [16], rw, [16], wsg, gq[2], gq[3], wsu, uq[2], uq[3], wsd, dq[2], dq[3],
            fm[0], fm[1], fm[2], fm[3], fm[4], fm[5], fm[6], fm[7], fm[8], fm[9], fm[10], x, [16],
            gq[0], gq[1], uq[0], uq[1], *sched, K, None, 28, MB, 256)
        assert len(bm) == 18 and tuple(bm[10].shape) == (MB, H) and bm[10].dtype == torch.float8_e4m3fn
        assert tuple(bm[13].shape) == (E_l, I, H)


def test_stage_copies_unless_the_value_already_is_the_buffer():
    from mok.functional import _stage
    buf = torch.zeros(4, 8)
    _stage(buf, buf)                                   # same tensor: nothing to do
    assert not buf.any()
    _stage(buf, torch.ones(4, 8))
    assert torch.equal(buf, torch.ones(4, 8))
    base = torch.zeros(2, 4, 8)
    _stage(base[0], base[0])                           # a view that is the buffer
    _stage(buf, base.view(-1)[:32].view(4, 8))         # same bytes elsewhere: copied
    assert not buf.any()
    wide = torch.arange(64.0).view(4, 16)
    _stage(buf, wide[:, :8])                           # same start address but another stride: copied, not aliased
    assert torch.equal(buf, wide[:, :8])


def test_functional_runs_operator_bodies_directly_only_in_plain_eager_mode():
    """`ops.call` skips the dispatcher in plain eager mode (same errors, version counters of mutated arguments still
    bumped) and goes through the registered operator under a dispatch mode, for subclasses and for tensors that
    require grad."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from mok import ops
    t = torch.zeros(4)
    assert ops._plain_eager((t, 3, [1, 2], None))
    assert not ops._plain_eager((torch.nn.Parameter(t),))
    assert not ops._plain_eager((t.clone().requires_grad_(),))
    with FakeTensorMode():
        assert not ops._plain_eager((t,))
    assert set(ops._EAGER) >= {ops.all_gather_top_experts, ops.barrier_all, ops.schedule, ops.fwd_epilogue, ops.bwd_epilogue,
                               ops.dispatch_mlp_swiglu_combine_fwd_bf16, ops.dispatch_mlp_swiglu_combine_bwd_bf16}
    assert ops._EAGER[ops.barrier_all][1] == (0, 3) and ops._EAGER[ops.dispatch_mlp_swiglu_combine_fwd_bf16][1] == (2,)
    # the body's own validation error, raised without a device in sight
    with pytest.raises(ValueError, match="CUDA"):
        ops.call(ops.barrier_all, torch.zeros(1, dtype=torch.int32), [1], 0, torch.zeros(1, dtype=torch.int32))

    seen = []

    @ops._op("mok_test::bump", mutates_args=("buf",))
    def bump(buf: torch.Tensor, by: int) -> None:
        seen.append(by)
        buf.add_(by)

    buf = torch.zeros(2)
    v0 = buf._version
    ops.call(bump, buf, 2)
    assert seen == [2] and buf._version > v0 and float(buf[0]) == 2.0
