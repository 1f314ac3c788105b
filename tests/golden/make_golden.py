"""Generate the golden fixtures in this directory by running the reference's own
pure-PyTorch implementation (its tests/utils.py) on CPU.

    python tests/golden/make_golden.py /path/to/reference

The reference file is loaded by path (it imports only torch); nothing of it is
copied.  Inputs come from oracle.mok_oracle.make_inputs (seeded CPU generators),
so a fixture stores outputs plus a checksum of the inputs they belong to.
gloo rejects the 2-D output tensor the reference passes to
all_gather_into_tensor (tests/utils.py:268,358-359), so that one call is wrapped
to flatten its arguments; the reference code itself is untouched.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import mok_oracle as O  # noqa: E402


def load_reference(path: str):
    spec = importlib.util.spec_from_file_location("ref_utils", os.path.join(path, "tests", "utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    real = dist.all_gather_into_tensor

    def flat_all_gather(out, inp, group=None, async_op=False):
        return real(out.view(-1), inp.reshape(-1), group=group, async_op=async_op)
    mod.dist.all_gather_into_tensor = flat_all_gather
    return mod


def u16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def checksum(t: torch.Tensor) -> int:
    b = t.contiguous().view(torch.uint8).numpy().reshape(-1).astype(np.uint64)
    return int((b * (np.arange(b.size, dtype=np.uint64) % 251 + 1)).sum() % (1 << 61))


SCHEDULE_CASES = [  # (name, R, T, K, E_l, factor, pattern)
    ("r1", 1, 512, 2, 8, 2, "random"),
    ("r2", 2, 512, 4, 4, 2, "random"),
    ("r4", 4, 512, 2, 2, 2, "random"),
    ("r8", 8, 512, 8, 4, 4, "random"),
    ("r4_mod", 4, 512, 1, 1, 2, "t_mod_R"),      # hand-built pattern of the reference's test_ops.py:200-226
    ("r4_skew", 4, 768, 3, 3, 4, "skew"),
    ("r2_empty", 2, 512, 2, 4, 2, "empty_expert"),
]


def schedule_topk(R, T, K, E_l, pattern, seed=11):
    E = E_l * R
    rng = np.random.default_rng(seed)
    if pattern == "t_mod_R":
        return np.tile((np.arange(T) % R).astype(np.int32)[None, :, None], (R, 1, 1))
    logits = rng.standard_normal((R, T, E)).astype(np.float32)
    if pattern == "skew":
        logits += -1.2 * np.log(np.arange(1, E + 1, dtype=np.float32))
    if pattern == "empty_expert":
        logits[:, :, 1] = -1e9
    return np.argsort(-logits, axis=-1, kind="stable")[:, :, :K].astype(np.int32)


def gen_single_process(ref, out):
    # --- schedule
    for name, R, T, K, E_l, factor, pattern in SCHEDULE_CASES:
        topk = schedule_topk(R, T, K, E_l, pattern)
        C = T * K * factor
        for rank in sorted({0, R - 1}):
            pr, pt, nt, tpe = ref.run_schedule_reference(torch.from_numpy(topk), E_l, C, rank)
            key = f"sched_{name}_rank{rank}"
            out[key + "_peer_rank"] = pr.numpy()
            out[key + "_peer_token_idx"] = pt.numpy()
            out[key + "_num_tokens"] = nt.numpy()
            out[key + "_tokens_per_expert"] = tpe.numpy()
    # --- quantiser
    g = torch.Generator().manual_seed(3)
    for name, shape, scale in (("q2d", (128, 256), 1.0), ("q3d", (2, 128, 128), 0.02), ("qwide", (256, 128), 30.0)):
        x = (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)
        q, s, qt, st = ref.run_mxfp8_quantize_reference(x, True, True)
        out[f"{name}_in"] = u16(x)
        out[f"{name}_fp8"] = q.view(torch.uint8).numpy()
        out[f"{name}_sc"] = s.numpy()
        out[f"{name}_fp8_t"] = qt.view(torch.uint8).numpy()
        out[f"{name}_sc_t"] = st.numpy()
    # --- swiglu + epilogues
    gate = (torch.randn(64, 128, generator=g) * 3).to(torch.bfloat16)
    up = (torch.randn(64, 128, generator=g) * 3).to(torch.bfloat16)
    out["swiglu_gate"], out["swiglu_up"] = u16(gate), u16(up)
    out["swiglu_none"] = u16(ref.run_swiglu_reference(gate, up, None))
    out["swiglu_clamp4"] = u16(ref.run_swiglu_reference(gate, up, 4.0))
    y = torch.randn(512, 256, generator=g).to(torch.bfloat16)
    comb = torch.randn(512 * 3, 256, generator=g).to(torch.bfloat16)
    w = torch.softmax(torch.randn(512, 3, generator=g), -1)
    out["epi_y"], out["epi_comb"], out["epi_w"] = u16(y), u16(comb), w.numpy()
    out["epi_fwd"] = u16(ref.run_fwd_epilogue_reference(y, comb, w))
    out["epi_bwd"] = u16(ref.run_bwd_epilogue_reference(y, comb))


LAYER_CASES = [  # (name, R, T, H, I, E, K, routing, limit)
    ("l1", 1, 512, 256, 256, 4, 2, "router", None),
    ("l1c", 1, 512, 256, 256, 4, 2, "gaussian", 1.0),
    ("l2", 2, 512, 256, 256, 4, 2, "gaussian", None),
]
LAYER_OUT = ("output", "d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
             "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def layer_worker(rank, world, ref_path, case, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // world))
    ref = load_reference(ref_path)
    name, R, T, H, I, E, K, routing, limit = case
    inp = O.make_inputs(R=R, T=T, H=H, I=I, E=E, K=K, seed=5, routing=routing)[rank]
    res = ref.run_reference_bf16(inp.x, inp.top_experts, inp.router_weights,
                                 inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down,
                                 inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down,
                                 inp.grad_output, limit)
    d = {}
    for k, t in zip(LAYER_OUT, res):
        t = t.detach()
        if k.startswith("d_w_routed"):
            t = t[:, ::4]               # every 4th row keeps the file small
        d[f"layer_{name}_rank{rank}_{k}"] = t.float().numpy() if t.dtype == torch.float32 else u16(t)
    d[f"layer_{name}_rank{rank}_input_checksum"] = np.array(
        [checksum(inp.x), checksum(inp.top_experts), checksum(inp.w_routed_gate), checksum(inp.grad_output)], np.int64)
    ret[rank] = d
    dist.destroy_process_group()


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of cursor/mixture-of-kittens>")
    ref_path = sys.argv[1]
    torch.manual_seed(0)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29611")
    dist.init_process_group("gloo", rank=0, world_size=1)
    ref = load_reference(ref_path)
    out: dict[str, np.ndarray] = {}
    gen_single_process(ref, out)
    dist.destroy_process_group()
    np.savez_compressed(os.path.join(HERE, "ops_golden.npz"), **out)

    layer: dict[str, np.ndarray] = {}
    for i, case in enumerate(LAYER_CASES):
        world = case[1]
        with mp.Manager() as mgr:
            ret = mgr.dict()
            mp.spawn(layer_worker, args=(world, ref_path, case, 29620 + i, ret), nprocs=world, join=True)
            for d in ret.values():
                layer.update(d)
    np.savez_compressed(os.path.join(HERE, "layer_golden.npz"), **layer)
    print("wrote", {k: os.path.getsize(os.path.join(HERE, k)) for k in ("ops_golden.npz", "layer_golden.npz")})


if __name__ == "__main__":
    main()
