"""The benchmark's stock-PyTorch baseline (all_to_all_single + grouped_mm + autograd) computes the same layer
as the oracle: two gloo ranks on CPU, outputs and gradients within the BF16 tolerance."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mok_oracle as O

GRADS = ("d_x", "d_router_weights", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down",
         "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down")


def _worker(rank, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=2)
    import bench
    ranks = O.make_inputs(R=2, T=256, H=128, I=64, E=4, K=2, seed=5, routing="gaussian")
    me = ranks[rank]
    leaves = [me.x.clone().requires_grad_(True), me.router_weights.clone().requires_grad_(True)]
    leaves += [w.clone().requires_grad_(True) for w in (me.w_shared_gate, me.w_shared_up, me.w_shared_down,
                                                        me.w_routed_gate, me.w_routed_up, me.w_routed_down)]
    out = bench.torch_all_to_all_layer(dist.group.WORLD, leaves[0], me.top_experts, leaves[1], *leaves[2:])
    grads = torch.autograd.grad(out, leaves, me.grad_output)
    ret[rank] = (out.detach(), [g.detach() for g in grads])
    dist.destroy_process_group()


def test_torch_all_to_all_layer_matches_the_oracle():
    ref = O.layer_forward_backward(O.make_inputs(R=2, T=256, H=128, I=64, E=4, K=2, seed=5, routing="gaussian"))
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(29733, ret), nprocs=2, join=True)
        for r in range(2):
            out, grads = ret[r]
            amax, rel = O.error_stats(ref[r]["output"], out)
            assert amax <= O.BF16_TOLERANCE[0] and rel <= O.BF16_TOLERANCE[1], ("output", r, amax, rel)
            for name, g in zip(GRADS, grads):
                amax, rel = O.error_stats(ref[r][name], g)
                assert amax <= O.BF16_TOLERANCE[0] and rel <= O.BF16_TOLERANCE[1], (name, r, amax, rel)
