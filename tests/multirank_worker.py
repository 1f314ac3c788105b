"""Worker of the multi-GPU parity test: run under torch.distributed.run, one rank per GPU.
Each rank computes the oracle for all ranks on CPU (same seeds everywhere), runs the layer
through mok.functional with expert parallelism over the ranks, and compares its own share."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    sys.path.insert(0, p)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from oracle import mok_oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from mok import _C, functional as F
    report = {"rank": rank, "world": world, "checks": {}}
    ok = True
    for case, (T, H, I, E_l, K, routing, limit) in enumerate([(512, 512, 256, 4, 2, "gaussian", None),
                                                             (1024, 256, 384, 3, 4, "zipf", 2.0)]):
        E = E_l * world
        ranks = O.make_inputs(R=world, T=T, H=H, I=I, E=E, K=K, seed=40 + case, routing=routing)
        factor = max(2, world)
        ref = O.layer_forward_backward(ranks, swiglu_limit=limit, schedule_capacity_factor=factor)[rank]
        inp = O.RankInputs(**{k: getattr(ranks[rank], k).to(dev) for k in ranks[rank].__dataclass_fields__})
        cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=T * K * factor, schedule_capacity_multiplier=1.0)
        ws = F.get_workspace(cfg, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
        for rep in range(2):       # twice: barrier targets and buffers are reused across steps
            sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
            out, ctx = F.forward(cfg, ws, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
                                 inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down, limit)
            grads = F.backward(cfg, ws, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate,
                               inp.w_shared_up, inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up,
                               inp.w_routed_down, limit)
        torch.cuda.synchronize()
        status = _C.check_status()
        checks = {"status": status}
        ok &= status == 0
        exact = bool((sched.peer_rank.cpu().numpy() == ref["peer_rank"]).all()
                     and (sched.peer_token_idx.cpu().numpy() == ref["peer_token_idx"]).all()
                     and (sched.tokens_per_expert.cpu().numpy() == ref["tokens_per_expert"]).all())
        checks["schedule_exact"] = exact
        ok &= exact
        N = int(ref["num_tokens"][0])
        xr = bool(torch.equal(ctx.x_routed[:N].cpu(), ref["x_routed"]))
        checks["dispatch_exact"] = xr
        ok &= xr
        names = ("output", "d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
                 "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")
        for name, got in zip(names, (out, *grads)):
            mx, rel = O.error_stats(ref[name], got.cpu())
            good = bool(np.isfinite(mx) and mx <= O.BF16_TOLERANCE[0] and rel <= O.BF16_TOLERANCE[1])
            checks[name] = [mx, rel, good]
            ok &= good
        report["checks"][f"case{case}"] = checks
        if case == 0:
            # the same layer with the routed experts in MXFP8, against the oracle's MXFP8 dataflow
            from mok import ops
            refq = O.layer_forward_backward(ranks, swiglu_limit=limit, schedule_capacity_factor=factor, mxfp8=True)[rank]
            qg, qu, qd = (ops.mxfp8_quantize(w, True, True) for w in (inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down))
            sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
            out, ctx = F.forward(cfg, ws, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
                                 inp.w_shared_down, (qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]), limit)
            grads = F.backward(cfg, ws, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate,
                               inp.w_shared_up, inp.w_shared_down, qg, qu, (qd[2], qd[3]), limit)
            torch.cuda.synchronize()
            mchecks = {"status": _C.check_status()}
            ok &= mchecks["status"] == 0
            for name, got in zip(names, (out, *grads)):
                mx, rel = O.error_stats(refq[name], got.cpu())
                good = bool(np.isfinite(mx) and mx <= 1.0 and rel <= 0.03)
                mchecks[name] = [mx, rel, good]
                ok &= good
            report["checks"]["case0_mxfp8"] = mchecks
            # both precisions again with macrobatches of 512 rows: the forward walks several of them, the backward
            # replays the later ones with a second round of peer pulls
            cfg_mb = F.MoKConfig(minibatch_size=256, macrobatch_size=512, schedule_capacity_multiplier=1.0)
            ws_mb = F.get_workspace(cfg_mb, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
            assert N > 512
            for label, wts, bwd_wts, want, tol_abs, tol_rel in (
                    ("case0_macrobatches_bf16", (inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down),
                     (inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down), ref, O.BF16_TOLERANCE[0], O.BF16_TOLERANCE[1]),
                    ("case0_macrobatches_mxfp8", ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1])), (qg, qu, (qd[2], qd[3])), refq, 1.0, 0.03)):
                sched = F.build_schedule(ws_mb, cfg_mb, inp.top_experts, num_local_experts=E_l)
                out, ctx = F.forward(cfg_mb, ws_mb, sched, inp.x, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
                                     inp.w_shared_down, *wts, limit)
                grads = F.backward(cfg_mb, ws_mb, sched, ctx, inp.grad_output, inp.x, inp.router_weights, inp.w_shared_gate,
                                   inp.w_shared_up, inp.w_shared_down, *bwd_wts, limit)
                torch.cuda.synchronize()
                rchecks = {"status": _C.check_status()}
                ok &= rchecks["status"] == 0
                for name, got in zip(names, (out, *grads)):
                    mx, rel = O.error_stats(want[name], got.cpu())
                    good = bool(np.isfinite(mx) and mx <= tol_abs and rel <= tol_rel)
                    rchecks[name] = [mx, rel, good]
                    ok &= good
                report["checks"][label] = rchecks
    report["ok"] = bool(ok)
    out_dir = os.environ.get("MOKB_TEST_OUT", "/tmp")
    with open(os.path.join(out_dir, f"multirank_rank{rank}.json"), "w") as f:
        json.dump(report, f)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
