"""Benchmark of the MoE layer hot path: build_schedule + forward + backward per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c4|c5|c2r|small] [--graph]
                    [--trace FILE] [--comm-sms S] [--minibatch M] [--no-mxfp8] [--no-torch-baseline] [--kernel-only]

For N > 1 launch under torch.distributed.run with one rank per GPU (RANK / LOCAL_RANK /
WORLD_SIZE / MASTER_* from the environment).  Rank 0 prints ONE JSON line.

Workload (default "c2"): 16384 tokens per rank, hidden 7168, 256 routed experts in total
(256 / N per rank) + one shared expert, top-8, expert width 2048 SwiGLU, balanced Gaussian
routing, BF16, minibatch 8192, capacity multiplier 0.5 -- synthetic data of that shape.
Per-GPU work is fixed as N grows (weak scaling).

  value      tokens/s over all ranks with the step's inputs already resident in HBM
  e2e        the same through mok.functional with the inputs in pinned HOST memory: host->device
             copies of x, top_experts, router_weights, grad_output and a device->host read of
             the result checksums are inside the timed region (double-buffered over two workspaces;
             e2e.serial: the copies on the compute stream before each step)
  parity     small multi-rank cases against the CPU oracle on every rank, run before anything is
             timed; a mismatch ends the run with a non-zero exit code
  in_step    GEMM time inside one traced step and the algorithmic TFLOP/s that corresponds to it
  ep8_share_1gpu  (1 GPU) one rank's share of the EP=8 run (32 experts), the anchor for 1 -> 8 scaling
  roofline   the dominant kernel (routed gate/up grouped GEMM with fused SwiGLU): algorithmic
             FLOPs per launch / its mean launch time (CUDA events, timed alone) over the
             measured cuBLAS BF16 burst peak of this pool (MEASURED_PEAKS.json)
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch path) on a bounded sample
  mxfp8      the same step with the routed experts in block-scaled E4M3 (+ its dominant kernel alone and
             cuBLASLt's block-scaled GEMM measured in the same run as a reference point)
  comm       (N > 1) dispatch and combine alone: NVLink GB/s per GPU and direction
  torch_all_to_all  the same layer in stock PyTorch (all_to_all_single + grouped_mm + autograd), BF16
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

WORKLOADS = {
    # name: (tokens per rank, hidden, intermediate, total experts, topk, minibatch, capacity multiplier, routing)
    "c2": (16384, 7168, 2048, 256, 8, 8192, 0.5, "gaussian"),
    "c1": (1024, 1024, 512, 8, 2, 256, 0.5, "router"),
    "c4": (16384, 4096, 1536, 128, 8, 8192, 1.0, "zipf"),
    "c5": (16384, 5120, 1408, 64, 6, 8192, 0.5, "gaussian"),
    "c2r": (16384, 7168, 2048, 32, 8, 8192, 0.5, "gaussian"),    # one rank's share of c2 at EP=8 (32 experts), without the NVLink part
    "small": (4096, 2048, 1024, 32, 4, 2048, 0.5, "gaussian"),   # for profiler captures: a few GB on the device
}
METRIC = "moe_layer_fwd_bwd_tokens_per_s"


def layer_flops(T, K, H, I):
    """fwd + bwd algorithmic FLOPs per rank: 18 * T * (K + 1) * H * I (shared expert included,
    padding and replay not counted) -- the reference's formula, benchmarks/utils.py:19-23."""
    return 18.0 * T * (K + 1) * H * I


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def sustained_peak():
    """cuBLAS bf16 in a seconds-long loop under the power cap (the regime of a kernel inside a step)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        if d.get("bf16_tflops_sustained"):
            return float(d["bf16_tflops_sustained"]), "measured"
    return 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.error = None
        self._nvml_handle = None

    def _nvml_sample(self):
        import pynvml
        h = self._nvml_handle
        bits = {"hw_slowdown": pynvml.nvmlClocksEventReasonHwSlowdown,
                "hw_thermal_slowdown": pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": pynvml.nvmlClocksEventReasonSwThermalSlowdown,
                "sw_power_cap": pynvml.nvmlClocksEventReasonSwPowerCap}
        sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
        mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
        try:
            pw = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:
            pw = 0.0
        r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
        flags = ["Active" if r & bits[n] else "Not Active" for n in
                 ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")]
        self.lines.append(", ".join([str(sm), str(mx), f"{pw:.1f}", *flags]))

    def _nvml_loop(self):
        # NVML from a thread: no process start-up, so even a 200 ms timed region gets samples
        failures = 0
        while not self._stop.is_set() and failures < 50:
            try:
                self._nvml_sample()
            except Exception as e:          # a transient NVML error must not end the sampling
                self.error = f"{type(e).__name__}: {e}"
                failures += 1
            self._stop.wait(0.02)

    def __enter__(self):
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self._nvml_handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return self
        except Exception as e:
            self.error = f"{type(e).__name__}: {e}"
            self._nvml_handle = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        self._stop.set()
        if not self.lines and self._nvml_handle is not None:
            try:                       # the sampling thread never ran: one reading right at the end of the region
                self._nvml_sample()
            except Exception as e:
                self.error = f"{type(e).__name__}: {e}"
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "error": self.error}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_oracle_sample(H, I, K, tokens=None):
    """One fwd+bwd of the CPU oracle on a bounded sample with the workload's per-token cost: K experts,
    top-K = K (every token visits K experts + the shared one).  `tokens` defaults to as many as make about
    15 TFLOP (10-20 s on a 16-core host), in multiples of 512.  Returns (tokens, experts, seconds)."""
    from oracle import mok_oracle as O
    Es = K
    Ts = tokens or int(min(8192, max(512, round(1.5e13 / layer_flops(1, K, H, I) / 512) * 512)))
    ranks = O.make_inputs(R=1, T=Ts, H=H, I=I, E=Es, K=K, seed=0, routing="gaussian")
    t0 = time.perf_counter()
    O.layer_forward_backward(ranks)
    dt = time.perf_counter() - t0
    return Ts, Es, dt


def host_threads():
    """All the host cores this process may use.  torch.distributed.run exports OMP_NUM_THREADS=1 to its workers,
    which would make the CPU arm an order of magnitude slower than the machine allows."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path (the oracle port of its PyTorch code) on the host cores, rank 0
    only.  Each step is one fwd+bwd on a bounded sample of the workload (same FLOPs per token); the sample is sized
    from a probe so that warm-up + steps end within about three minutes whatever the core count."""
    if rank != 0:
        return
    cores = host_threads()
    T, H, I, E, K, mb, mult, routing = WORKLOADS[args.workload]
    n_samples = args.warmup + args.steps
    _, _, probe_s = cpu_oracle_sample(H, I, K, tokens=512)          # also pages the host libraries in
    _, _, probe_s = cpu_oracle_sample(H, I, K, tokens=512)
    per_sample_s = min(10.0, 180.0 / n_samples)
    Ts = int(min(8192, max(512, round(per_sample_s / probe_s * 512 / 512) * 512)))
    times = []
    for i in range(n_samples):
        Ts, Es, dt = cpu_oracle_sample(H, I, K, tokens=Ts)
        if i >= args.warmup:
            times.append(dt)
    ms = 1000.0 * sum(times) / len(times)
    value = Ts / (ms / 1000.0)
    sample = f"{Ts} tokens x top-{K} over {Es} experts + shared expert, H={H}, I={I}, fwd+bwd (same FLOPs per token as the workload)"
    cfg = workload_config(args.workload, args.gpus)
    cfg["sample"] = {"tokens": Ts, "experts": Es, "topk": K, "hidden": H, "intermediate": I, "ep_size": 1,
                     "note": "the CPU arm times this bounded sample, not the full workload; tokens/s is per-token cost"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


class _AllToAllRows(torch.autograd.Function):
    """`dist.all_to_all_single` over dim 0 with the reverse exchange as its gradient."""

    @staticmethod
    def forward(ctx, inp, out_splits, in_splits, group):
        ctx.args = (out_splits, in_splits, group)
        out = inp.new_empty((sum(out_splits),) + tuple(inp.shape[1:]))
        dist.all_to_all_single(out, inp.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        out_splits, in_splits, group = ctx.args
        gin = grad.new_empty((sum(in_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(gin, grad.contiguous(), in_splits, out_splits, group=group)
        return gin, None, None, None


def torch_all_to_all_layer(group, x, top_experts, router_weights, wsg, wsu, wsd, wrg, wru, wrd):
    """The same layer written with stock PyTorch ops and NCCL (or gloo) collectives: count routes per expert,
    exchange the counts, sort the routes by expert, `all_to_all_single` the token rows to the experts' ranks,
    `torch._grouped_mm` per local expert, send the rows back, weighted sum at home.  This is the "torch all-to-all"
    baseline the reference compares itself with (its benchmarks/bench_nccl_torch.py:36-229), restated without TorchAO;
    autograd provides the backward pass.  Split sizes are read on the host, as that baseline does."""
    import torch.nn.functional as Fn
    R = dist.get_world_size(group)
    T, H = x.shape
    K = top_experts.shape[1]
    E_l = wrg.shape[0]
    E = E_l * R
    flat = top_experts.reshape(-1)
    order = torch.argsort(flat, stable=True)                   # routes by expert, hence by destination rank
    counts = torch.bincount(flat, minlength=E)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)   # [R, E_l]: rows from rank r for local expert e
    recv_mat = recv_counts.view(R, E_l)
    send_splits = counts.view(R, E_l).sum(1).tolist()
    recv_splits = recv_mat.sum(1).tolist()
    rows = _AllToAllRows.apply(x[order // K], recv_splits, send_splits, group)
    # received rows are grouped by (source rank, expert): regroup by expert
    expert_of_row = torch.repeat_interleave(torch.arange(E_l, device=x.device).repeat(R), recv_mat.reshape(-1))
    by_expert = torch.argsort(expert_of_row, stable=True)
    xe = rows[by_expert]
    offs = recv_mat.sum(0).cumsum(0).to(torch.int32)
    gate = torch._grouped_mm(xe, wrg.transpose(1, 2), offs=offs)
    up = torch._grouped_mm(xe, wru.transpose(1, 2), offs=offs)
    y = torch._grouped_mm(Fn.silu(gate) * up, wrd.transpose(1, 2), offs=offs)
    back = _AllToAllRows.apply(y[torch.argsort(by_expert)], send_splits, recv_splits, group)
    routed = back[torch.argsort(order)].view(T, K, H)
    out = torch.bmm(router_weights.to(routed.dtype).unsqueeze(1), routed).squeeze(1)
    shared = (Fn.silu(x @ wsg.t()) * (x @ wsu.t())) @ wsd.t()
    return out + shared


def time_torch_all_to_all(group, timed, steps, warmup, x, te, rw, gy, weights):
    """fwd + bwd of `torch_all_to_all_layer` (gradients of x, the router weights and all six weight tensors)."""
    leaves = [x.detach().clone().requires_grad_(True), rw.detach().clone().requires_grad_(True)]
    leaves += [w_.detach().requires_grad_(True) for w_ in weights]

    def step():
        out = torch_all_to_all_layer(group, leaves[0], te, leaves[1], *leaves[2:])
        return torch.autograd.grad(out, leaves, gy)
    for _ in range(warmup):
        step()
    return timed(step, steps) / steps


def cublaslt_mxfp8_tflops(device, seconds=1.0):
    """Library reference point for the MXFP8 numbers: an 8192^3 block-scaled E4M3 GEMM (E8M0 scale per 32 along K)
    through torch._scaled_mm (cuBLASLt), as a burst of 20 calls and as a loop of about `seconds`.
    Returns (burst TFLOP/s, sustained TFLOP/s) or a string saying why it could not run."""
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        sa = torch.full((n, n // 32), 127, dtype=torch.uint8, device=device).view(torch.float8_e8m0fnu)
        sb = torch.full((n, n // 32), 127, dtype=torch.uint8, device=device).view(torch.float8_e8m0fnu)

        def mm():
            return torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        for _ in range(3):
            mm()
        torch.cuda.synchronize()
        flops = 2.0 * n * n * n

        def run(iters):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(iters):
                mm()
            end.record()
            torch.cuda.synchronize()
            return flops * iters / (start.elapsed_time(end) / 1000.0) / 1e12
        burst = run(20)
        sustained = run(max(20, int(seconds * burst * 1e12 / flops)))
        return burst, sustained
    except Exception as e:
        return f"{type(e).__name__}: {str(e)[:160]}"


def workload_config(name, n):
    T, H, I, E, K, mb, mult, routing = WORKLOADS[name]
    return {"workload": f"{name}: MoE layer fwd+bwd, {T} tokens/rank, hidden {H}, {E} routed experts ({E // n}/rank) + 1 shared, "
                        f"top-{K}, expert width {I} SwiGLU, {routing} routing, EP={n}",
            "tokens_per_rank": T, "hidden": H, "intermediate": I, "experts": E, "topk": K, "minibatch_size": mb,
            "schedule_capacity_multiplier": mult, "ep_size": n, "l2": "inputs_larger_than_l2",
            "staging": "activations are produced in the workspace's symmetric buffers (no staging copies)"}


class Problem:
    """One workload on this rank: inputs in pinned host memory, weights and the workspace on the device, and the
    BF16 / MXFP8 step functions (build_schedule + forward + backward through mok.functional)."""

    def __init__(self, name, args, rank, world, device, group, *, tokens=None, minibatch=None, host_inputs=True):
        from mok import functional as F
        self.F, self.name, self.rank, self.world, self.device, self.group = F, name, rank, world, device, group
        T, H, I, E, K, mb, mult, routing = WORKLOADS[name]
        T = tokens or T
        if minibatch or args.minibatch:
            mb = minibatch or args.minibatch
        assert E % world == 0
        E_l = E // world
        MB = int(math.ceil((T * K + E_l * 256) / mb) * mb)
        self.T, self.H, self.I, self.E, self.K, self.mb, self.E_l, self.MB = T, H, I, E, K, mb, E_l, MB
        kw = dict(minibatch_size=mb, macrobatch_size=MB, schedule_capacity_multiplier=mult)
        if args.comm_sms:
            kw.update(fwd_num_comm_sms=args.comm_sms, bwd_num_comm_sms=args.comm_sms)
        self.cfg = F.MoKConfig(**kw)
        # per-step inputs: in pinned host memory for the end-to-end legs; sweeps generate them on the device
        gen_dev = torch.device("cpu") if host_inputs else device
        g = torch.Generator(device=gen_dev).manual_seed(1000 + rank)
        pin = (lambda t: t.pin_memory()) if host_inputs else (lambda t: t)
        self.x_h = pin(torch.randn(T, H, generator=g, device=gen_dev).to(torch.bfloat16))
        self.gy_h = pin(torch.randn(T, H, generator=g, device=gen_dev).to(torch.bfloat16))
        logits = torch.randn(T, E, generator=g, device=gen_dev)
        if routing == "zipf":
            perm = torch.randperm(E, generator=torch.Generator().manual_seed(7))
            bias = torch.empty(E)
            bias[perm] = -1.2 * torch.log(torch.arange(1, E + 1, dtype=torch.float32))
            logits = logits + bias.to(gen_dev)
        vals, idx = torch.topk(logits, K, dim=1)
        self.te_h = pin(idx.to(torch.int64))
        self.rw_h = pin(torch.softmax(vals.float(), -1))
        del logits
        gd = torch.Generator(device=device).manual_seed(2000 + rank)

        def w(*shape):
            t = torch.empty(*shape, dtype=torch.bfloat16, device=device)
            t.normal_(0.0, 0.02, generator=gd)
            return t
        self.shared = (w(I, H), w(I, H), w(H, I))
        self.routed = (w(E_l, I, H), w(E_l, I, H), w(E_l, H, I))
        self.ws = F.get_workspace(self.cfg, group, device=device, num_local_tokens=T, hidden_size=H, topk=K)
        # the step's activations live where the layer wants them: in the workspace's symmetric buffers, so
        # functional.forward / backward skip their staging copies (the copies the reference marks as removable)
        self.x_d, self.gy_d, self.rw_d = self.ws.x_buffer, self.ws.d_y_buffer, self.ws.router_weight_buffer
        self.load_resident()
        self.te_d = self.te_h.to(device)
        self.mid = None                     # event recorded between forward and backward when set
        self.q = None

    def load_resident(self):
        self.x_d.copy_(self.x_h)
        self.gy_d.copy_(self.gy_h)
        self.rw_d.copy_(self.rw_h)

    def flops(self):
        return layer_flops(self.T, self.K, self.H, self.I)

    def step(self, x=None, te=None, rw=None, gy=None, ws=None):
        F = self.F
        ws = ws or self.ws
        x, te, rw, gy = (self.x_d if x is None else x, self.te_d if te is None else te,
                         self.rw_d if rw is None else rw, self.gy_d if gy is None else gy)
        sched = F.build_schedule(ws, self.cfg, te, num_local_experts=self.E_l)
        out, ctx = F.forward(self.cfg, ws, sched, x, rw, *self.shared, *self.routed)
        if self.mid is not None:
            self.mid.record()
        grads = F.backward(self.cfg, ws, sched, ctx, gy, x, rw, *self.shared, *self.routed)
        return sched, out, grads

    def quantise_weights(self):
        from mok import ops
        if self.q is None:
            self.q = tuple(ops.mxfp8_quantize(w_, True, True) for w_ in self.routed)
        return self.q

    def step_mx(self):
        F = self.F
        qg, qu, qd = self.quantise_weights()
        sched = F.build_schedule(self.ws, self.cfg, self.te_d, num_local_experts=self.E_l)
        out, ctx = F.forward(self.cfg, self.ws, sched, self.x_d, self.rw_d, *self.shared, (qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
        if self.mid is not None:
            self.mid.record()
        return F.backward(self.cfg, self.ws, sched, ctx, self.gy_d, self.x_d, self.rw_d, *self.shared, qg, qu, (qd[2], qd[3]))


def make_timer(device):
    """timed(fn, steps) -> (total ms, [per-step ms]): `steps` calls bracketed by a barrier + synchronize on both sides,
    CUDA events on the launching stream after every step, each figure the maximum over ranks."""
    def timed(fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        ev[0].record()
        for i in range(steps):
            fn()
            ev[i + 1].record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([ev[0].elapsed_time(ev[-1])] + [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)],
                         dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t = t.tolist()
        return t[0], t[1:]
    return timed


def fwd_bwd_split(prob, fn, reps):
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    prob.mid = ev[1]
    f, b = [], []
    for _ in range(reps):
        torch.cuda.synchronize()
        ev[0].record()
        fn()
        ev[2].record()
        torch.cuda.synchronize()
        f.append(ev[0].elapsed_time(ev[1]))
        b.append(ev[1].elapsed_time(ev[2]))
    prob.mid = None
    return statistics.median(f), statistics.median(b)


def traced_step(_C, fn):
    """The launch timeline of one step; a first traced step is thrown away (it creates the timing events)."""
    recs = None
    for _ in range(2):
        torch.cuda.synchronize()
        dist.barrier()
        _C.trace_begin()
        fn()
        recs = _C.trace_end()
    return recs


def in_step_summary(recs, prefix, prob, real_rows, peak_tf):
    """GEMM time inside one traced step (sum of the launch intervals of this library's GEMM launchers) and the
    algorithmic TFLOP/s that corresponds to it; the gate/up kind (routed + shared) on its own as well."""
    gemm = [r for r in recs if r[0].startswith(prefix)]
    if not gemm:
        return None
    busy = sum(r[4] - r[3] for r in gemm)
    span = max(r[4] for r in recs) - min(r[3] for r in recs)
    out = {"step_ms_traced": span, "gemm_launches": len(gemm), "gemm_busy_ms": busy,
           "gemm_tflops": prob.flops() / (busy / 1000.0) / 1e12,
           "note": "algorithmic FLOPs (padding and replay not counted) over the GEMM launch intervals of one traced step"}
    # the routed forward is one persistent launch: gate/up + SwiGLU and the down projection of every window
    fr_ms = sum(r[4] - r[3] for r in gemm if r[0] == prefix + "_fwd_routed")
    out["fwd_routed_ms"] = fr_ms
    out["fwd_routed_tflops"] = 6.0 * real_rows * prob.H * prob.I / (fr_ms / 1000.0) / 1e12 if fr_ms > 0 else None
    if prefix == "gemm_bf16":
        out["gemm_frac_of_burst"] = out["gemm_tflops"] / peak_tf
        out["fwd_routed_frac_of_burst"] = out["fwd_routed_tflops"] / peak_tf if out["fwd_routed_tflops"] else None
    else:
        out["note"] += "; the BF16 shared expert's GEMMs are not in gemm_busy_ms, its FLOPs (1/(K+1) of the layer) are"
    return out


def gate_up_bytes(prob, padded_rows, experts_used):
    """Algorithmic HBM bytes of one routed gate/up + SwiGLU launch: A rows once, both weight matrices of every
    expert that has rows once, and the three outputs."""
    a = padded_rows * prob.H * 2
    wts = experts_used * 2 * prob.I * prob.H * 2
    outs = 3 * padded_rows * prob.I * 2
    return {"a_rows": a, "weights": wts, "outputs": outs, "total": a + wts + outs}


def fwd_routed_bytes(prob, padded_rows, experts_used):
    """Algorithmic HBM bytes of the routed forward launch: the gate/up part plus the down weights and the y rows
    (hidden is read back from L2 / HBM once)."""
    m = gate_up_bytes(prob, padded_rows, experts_used)
    m["weights"] += experts_used * prob.H * prob.I * 2
    m["hidden_reread"] = padded_rows * prob.I * 2
    m["outputs"] += padded_rows * prob.H * 2
    m["total"] = m["a_rows"] + m["weights"] + m["outputs"] + m["hidden_reread"]
    return m


def comm_alone(prob, sched, timed, _C, rank):
    """Dispatch (row pull) and combine (row push) kernels alone over the first macrobatch's rows, every rank at once.  The rate is
    the remote rows of the busiest rank (its inbound bytes when pulling, outbound when pushing) over the slowest rank's time."""
    # entries past num_tokens are not written by the schedule; the kernels below move the first macrobatch
    live = sched.peer_rank[: min(int(sched.num_tokens.item()), prob.MB)]
    whole = sched.peer_rank[: int(sched.num_tokens.item())]
    remote_t = torch.stack([((live >= 0) & (live != rank)).sum(), ((whole >= 0) & (whole != rank)).sum()]).to(torch.int64)
    dist.all_reduce(remote_t, op=dist.ReduceOp.MAX)              # the busiest rank: the time below is the slowest rank's
    remote, remote_step = (int(v) for v in remote_t.tolist())
    buf = torch.empty(prob.MB, prob.H, dtype=torch.bfloat16, device=prob.device)
    cap = sched.peer_rank.numel()
    ws, out = prob.ws, {"remote_rows": remote, "remote_rows_step": remote_step}
    for name, fn in (
        # (row window [0, MB) of the schedule: a rank with more rows than one macrobatch moves the first macrobatch)
        ("dispatch", lambda: _C.dispatch_rows_window(ws.x_buffer_ptrs, sched.peer_rank, sched.peer_token_idx, sched.num_tokens,
                                                     cap, 0, prob.MB, prob.K, prob.H, buf, index_limit=prob.T * prob.K)),
        ("combine", lambda: _C.combine_rows_window(buf, ws.combine_buffer_ptrs, sched.peer_rank, sched.peer_token_idx,
                                                   sched.num_tokens, cap, 0, prob.MB, prob.H, index_limit=prob.T * prob.K)),
    ):
        fn()
        ms = timed(fn, 5)[0] / 5
        gbs = remote * prob.H * 2 / (ms / 1000.0) / 1e9
        out[name] = {"ms": ms, "nvlink_gbs": gbs, "frac_of_900": gbs / 900.0, "frac_of_measured_770": gbs / 770.0}
    return out


def run_sweep(args, rank, world, device, group, timed, _C):
    """Config 4 (Zipf routing, multiplier 1.0) and the config-5 grid (tokens per rank x minibatch) at EP = world, BF16
    and MXFP8: ms per step, tokens/s/GPU, TFLOP/s/GPU and the NVLink rate of the communication phases.  One JSON
    line per cell on rank 0 (and in --sweep-out), inputs generated on the device."""
    from mok import functional as F
    cells = [("c4", None, None)] + [("c5", T, mb) for T in (4096, 16384, 65536) for mb in (2048, 8192, 16384)]
    if args.sweep != "all":
        cells = [c for c in cells if c[0] == args.sweep]
    lines = []
    last_T = None
    for name, T, mb in cells:
        if last_T is not None and T != last_T:
            F.clear_workspace_cache()
            torch.cuda.empty_cache()
        last_T = T
        prob = Problem(name, args, rank, world, device, group, tokens=T, minibatch=mb, host_inputs=False)
        cell = {"sweep": name, "n_gpus": world, "tokens_per_rank": prob.T, "minibatch_size": prob.mb, "hidden": prob.H,
                "intermediate": prob.I, "experts": prob.E, "topk": prob.K, "macrobatch_size": prob.MB}
        for label, fn in (("bf16", prob.step), ("mxfp8", prob.step_mx)):
            if label == "mxfp8" and args.no_mxfp8:
                continue
            for _ in range(3):
                fn()
            ms = statistics.median(timed(fn, args.steps)[1])
            cell[label] = {"ms_per_step": ms, "tokens_per_s_per_gpu": prob.T / (ms / 1000.0),
                           "tflops_per_gpu": prob.flops() / (ms / 1000.0) / 1e12}
        status = _C.check_status()
        cell["status"] = status
        sched, _, _ = prob.step()
        rows = int(sched.num_tokens.item())
        ranks_rows = torch.tensor([rows], dtype=torch.int64, device=device)
        allr = [torch.zeros_like(ranks_rows) for _ in range(world)]
        dist.all_gather(allr, ranks_rows)
        cell["padded_rows_per_rank"] = [int(t.item()) for t in allr]
        if world > 1:
            comm = comm_alone(prob, sched, timed, _C, rank)
            # bytes that cross NVLink in one step (forward pull + push, backward pull + push) over the step time
            step_bytes = 4.0 * comm["remote_rows_step"] * prob.H * 2
            comm["in_step_gbs_bf16"] = step_bytes / (cell["bf16"]["ms_per_step"] / 1000.0) / 1e9
            cell["comm"] = comm
        prob.q = None
        del prob, sched
        torch.cuda.empty_cache()
        lines.append(cell)
        if rank == 0:
            print(json.dumps(cell), flush=True)
    if rank == 0 and args.sweep_out:
        with open(args.sweep_out, "a") as f:
            for cell in lines:
                f.write(json.dumps(cell) + "\n")


def run_parity_leg(rank, world, device):
    """Small multi-rank cases against the CPU oracle on every rank, before anything is timed."""
    from tests.parity_cases import run_parity, summarise
    old = torch.get_num_threads()
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) // max(1, world)))
    except AttributeError:
        pass
    rep = run_parity(rank, world, device)
    torch.set_num_threads(old)
    reports = [None] * world
    dist.all_gather_object(reports, rep)
    return summarise(reports)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--minibatch", type=int, default=0, help="override the workload's minibatch_size (overlap window)")
    ap.add_argument("--comm-sms", type=int, default=0, help="override fwd/bwd_num_comm_sms")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity leg (small cases against the CPU oracle on every rank)")
    ap.add_argument("--no-mxfp8", action="store_true", help="skip the MXFP8 leg (reported under the key \"mxfp8\")")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end legs (sweeps; the line then has no e2e key)")
    ap.add_argument("--no-torch-baseline", action="store_true",
                    help="skip the stock-PyTorch all-to-all + grouped_mm baseline (reported under \"torch_all_to_all\")")
    ap.add_argument("--graph", action="store_true", help="1 GPU: also time the step replayed from a CUDA graph (always on for c1)")
    ap.add_argument("--no-share", action="store_true", help="skip the 1-GPU leg that runs one rank's EP=8 share of config 2")
    ap.add_argument("--trace", default="", help="write the launch timeline of one BF16 and one MXFP8 step of rank 0 to this file")
    ap.add_argument("--kernel-only", action="store_true", help="time only the dominant GEMM (profiler captures)")
    ap.add_argument("--sweep", default="", choices=["", "c4", "c5", "all"],
                    help="instead of the benchmark line: config 4 and / or the config-5 grid (tokens x minibatch) at EP = --gpus")
    ap.add_argument("--sweep-out", default="", help="append the sweep's JSON lines to this file")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if not args.kernel_only else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")

    from mok import _C

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29551")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    group = dist.group.WORLD
    timed = make_timer(device)
    peak_tf, peak_gbs, peak_kind = measured_peaks()

    # ---- parity first: a fast wrong answer is not a result
    parity = None
    if not (args.no_parity or args.kernel_only):
        parity = run_parity_leg(rank, world, device)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "parity": parity,
                                  "error": "the layer's results differ from the CPU oracle's; nothing was timed"}), flush=True)
            dist.destroy_process_group()
            raise SystemExit(1)
        from mok import functional as F
        F.clear_workspace_cache()
        torch.cuda.empty_cache()

    if args.sweep:
        run_sweep(args, rank, world, device, group, timed, _C)
        dist.destroy_process_group()
        return

    prob = Problem(args.workload, args, rank, world, device, group)
    T, H, I, E, K, E_l, MB = prob.T, prob.H, prob.I, prob.E, prob.K, prob.E_l, prob.MB
    ws = prob.ws
    x_h, gy_h, te_h, rw_h = prob.x_h, prob.gy_h, prob.te_h, prob.rw_h
    wrg, wru, wrd = prob.routed

    if args.kernel_only:
        sched = prob.F.build_schedule(ws, prob.cfg, prob.te_d, num_local_experts=E_l)
        torch.cuda.synchronize()
        kern = time_dominant_kernel(_C, sched, prob.x_d, wrg, wru, T, H, I, K, E_l, MB, args.steps, args.warmup, device, wrd=wrd)
        kern["wgrad_down"] = time_wgrad_kernel(_C, sched, T, H, I, E_l, MB, args.steps, args.warmup, device)
        if not args.no_mxfp8:
            from mok import ops
            qg, qu, qd = (ops.mxfp8_quantize(w_, True, False) for w_ in (wrg, wru, wrd))
            kern["mxfp8"] = time_dominant_kernel_mxfp8(_C, ops, sched, prob.x_d, qg, qu, T, H, I, E_l, MB, args.steps, args.warmup,
                                                       device, qd=qd)
        if rank == 0:
            print(json.dumps({"kernel_only": True, **kern}), flush=True)
        dist.destroy_process_group()
        return

    # ---- device-resident steps
    for _ in range(args.warmup):
        prob.step()
    torch.cuda.synchronize()
    assert _C.check_status() == 0, f"device status word set during warm-up: {_C.status_detail()}"
    launches_before = _C.launch_count()
    with ClockSampler(local_rank) as clocks:
        total_ms, per_step = timed(prob.step, args.steps)
    launches = _C.launch_count() - launches_before
    clock_summary = clocks.summary()
    if world > 1:      # every rank sampled its own GPU: the step runs at the pace of the slowest one
        per_rank = [None] * world
        dist.all_gather_object(per_rank, clock_summary.get("sm_mhz"))
        clock_summary["sm_mhz_per_rank"] = per_rank
    ms_per_step = total_ms / args.steps
    fwd_ms, bwd_ms = fwd_bwd_split(prob, prob.step, max(2, args.steps // 4))
    assert _C.check_status() == 0, f"device status word set during the timed region: {_C.status_detail()}"

    sched, _, _ = prob.step()
    real_rows = int((sched.peer_rank >= 0).sum().item())
    padded_rows = int(sched.num_tokens.item())
    experts_used = int((sched.tokens_per_expert > 0).sum().item())
    trace_lines = []
    rec_bf16 = traced_step(_C, prob.step)
    trace_lines += [("bf16",) + rec for rec in rec_bf16]
    in_step = {"bf16": in_step_summary(rec_bf16, "gemm_bf16", prob, real_rows, peak_tf)}

    # ---- end to end: inputs start in pinned host memory, result checksums come back to the host
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(prob, timed, args.steps, _C)
        prob.load_resident()              # the device-resident legs below read the symmetric buffers again

    # ---- roofline of the dominant kernel
    kern = time_dominant_kernel(_C, sched, prob.x_d, wrg, wru, T, H, I, K, E_l, MB, 5, 2, device, wrd=wrd)
    kern_gu = time_dominant_kernel(_C, sched, prob.x_d, wrg, wru, T, H, I, K, E_l, MB, 5, 2, device)
    model = fwd_routed_bytes(prob, padded_rows, experts_used)
    kern_per_rank = [None] * world        # the same launch on every rank's own rows and GPU, at the same time
    if world > 1:
        dist.all_gather_object(kern_per_rank, round(kern["tflops"], 1))
    else:
        kern_per_rank = [round(kern["tflops"], 1)]
    traffic, traffic_note = None, None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        ratio = tj.get("fwd_routed_gemm_dram_over_algorithmic_bytes")
        if ratio:
            traffic = ratio * model["total"]
            traffic_note = (f"algorithmic bytes of this launch x {ratio} = DRAM bytes / algorithmic bytes that ncu measured "
                            "for this kernel on the 'small' workload (profiles/traffic.json); not a capture of this launch")
    roofline = {"bound": "tensor", "kernel": "grouped_gemm_kernel<MODE_FWD> (routed gate/up + SwiGLU + down, one persistent launch)",
                "achieved": kern["tflops"], "peak": peak_tf, "unit": "TFLOP/s", "frac": kern["tflops"] / peak_tf,
                "peak_source": f"{peak_kind} cuBLAS bf16 burst", "traffic": traffic, "traffic_source": traffic_note,
                "algorithmic_bytes": model, "launch_ms": kern["ms"], "flops_per_launch": kern["flops_per_launch"],
                "rows": real_rows, "padded_rows": padded_rows,
                "tflops_on_padded_rows": kern["tflops"] * padded_rows / max(real_rows, 1),
                "tflops_per_rank": kern_per_rank,
                # `frac` is against the burst figure (the launch is timed alone); the timing loop itself runs for about a
                # second under the power cap, so the sustained figure is given beside it
                "frac_of_sustained": kern["tflops"] / sustained_peak()[0], "peak_sustained": sustained_peak()[0],
                "peak_sustained_source": f"{sustained_peak()[1]} cuBLAS bf16, back to back for seconds",
                "gate_up_launch_alone": {"ms": kern_gu["ms"], "tflops": kern_gu["tflops"], "frac": kern_gu["tflops"] / peak_tf,
                                         "note": "the gate/up + SwiGLU launch (mode 1) on the same rows: the launch that dominated before the forward became one launch"}}

    # ---- the communication phases alone: dispatch (row pull) and combine (row push) over all scheduled rows,
    # every rank at once, CUDA events, max over ranks.  Bytes over NVLink = rows whose home is another rank.
    comm = None
    if world > 1:
        comm = {"rows": padded_rows, "nvlink_peak_gbs_per_direction": 900.0, "measured_peer_copy_gbs": 770.0,
                **comm_alone(prob, sched, timed, _C, rank)}
        comm["in_step_gbs_bf16"] = 4.0 * comm["remote_rows_step"] * H * 2 / (ms_per_step / 1000.0) / 1e9

    # ---- the same step with the routed experts in MXFP8 (weights pre-quantised outside the step, as the reference does)
    mx = None
    if not args.no_mxfp8:
        from mok import ops
        mx = run_mxfp8_leg(prob, timed, args, _C, ops, sched, real_rows, peak_tf, trace_lines, in_step, rank, device)

    # ---- baseline: the same layer with stock PyTorch ops (all_to_all_single + grouped_mm + autograd), BF16
    tb = None
    if not args.no_torch_baseline:
        try:
            tb_steps = max(2, min(args.steps, 5))
            tb_ms = time_torch_all_to_all(group, lambda fn, n: timed(fn, n)[0], tb_steps, 2, prob.x_d, prob.te_d, prob.rw_d, prob.gy_d,
                                          (*prob.shared, *prob.routed))
            tb = {"value": T * world / (tb_ms / 1000.0), "unit": "tokens/s", "ms_per_step": tb_ms, "steps": tb_steps,
                  "tflops_per_gpu": prob.flops() / (tb_ms / 1000.0) / 1e12,
                  "note": "all_to_all_single (NCCL) + torch._grouped_mm + autograd, BF16, same inputs and weights"}
        except Exception as e:      # a library baseline must not take the benchmark down
            tb = {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}
        torch.cuda.empty_cache()

    # ---- 1 GPU, small workloads: the same step replayed from a CUDA graph (the launch-bound regime)
    graph_leg = None
    if world == 1 and (args.graph or args.workload == "c1"):
        graph_leg = run_graph_leg(prob, timed, args.steps, no_mxfp8=args.no_mxfp8)

    # ---- 1 GPU only: one rank's share of the EP=8 run of config 2 (32 local experts), the honest anchor for 1 -> 8 scaling
    share = None
    if world == 1 and args.workload == "c2" and not args.no_share:
        prob.q = None
        del prob, wrg, wru, wrd, sched, ws, kern
        torch.cuda.empty_cache()
        sp = Problem("c2r", args, rank, world, device, group)
        for _ in range(3):
            sp.step()
        s_ms = timed(sp.step, max(5, args.steps // 2))[1]
        share = {"workload": "c2r: config 2 with 32 routed experts (what one rank holds at EP=8), no NVLink",
                 "ms_per_step": statistics.median(s_ms), "tflops_per_gpu": sp.flops() / (statistics.median(s_ms) / 1000.0) / 1e12}
        if not args.no_mxfp8:
            for _ in range(3):
                sp.step_mx()
            m_ms = timed(sp.step_mx, max(5, args.steps // 2))[1]
            share["mxfp8_ms_per_step"] = statistics.median(m_ms)
            share["mxfp8_tflops_per_gpu"] = sp.flops() / (statistics.median(m_ms) / 1000.0) / 1e12
        assert _C.check_status() == 0, f"device status word set during the EP=8-share leg: {_C.status_detail()}"
        del sp
        torch.cuda.empty_cache()

    if rank == 0 and args.trace:
        with open(args.trace, "w") as f:
            f.write("# leg tag first_row stream begin_ms end_ms\n")
            for rec in trace_lines:
                f.write(" ".join(str(v) for v in rec) + "\n")

    if rank == 0:
        tokens = T * world
        flops = layer_flops(T, K, H, I)
        line = {
            "metric": METRIC, "value": tokens / (ms_per_step / 1000.0), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world),
            "median_ms_per_step": statistics.median(per_step),
            "tokens_per_s_per_gpu": T / (ms_per_step / 1000.0),
            "tflops_per_gpu": flops / (ms_per_step / 1000.0) / 1e12,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
            "roofline": roofline,
            "in_step": in_step,
            "gpu_launches": int(launches),
            "clocks": clock_summary,
        }
        if parity is not None:
            line["parity"] = parity
        if e2e is not None:
            line["e2e"] = {k: (tokens / (v / 1000.0) if k == "value" else v) for k, v in e2e.items()}
        if mx is not None:
            line["mxfp8"] = mx
        if comm is not None:
            line["comm"] = comm
        if tb is not None:
            line["torch_all_to_all"] = tb
        if share is not None:
            line["ep8_share_1gpu"] = share
        if graph_leg is not None:
            line["cuda_graph"] = graph_leg
        if world == 1 and not args.no_cpu_baseline:
            cores = host_threads()
            Ts, Es, dt = cpu_oracle_sample(H, I, K)
            line["cpu_baseline"] = {
                "value": Ts / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": f"{Ts} tokens x top-{K} over {Es} experts + shared expert, H={H}, I={I}, one fwd+bwd of the CPU oracle "
                          f"({dt:.1f} s; same FLOPs per token as the workload)"}
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def run_e2e(prob, timed, steps, _C):
    """The step through mok.functional with the four inputs in pinned HOST memory: host -> device copies (straight into
    the workspace's symmetric buffers) and a device -> host read of two checksums inside the timed region.  Returns
    {"value": ms per step (converted to tokens/s by the caller), ...}."""
    device = prob.device
    x_h, gy_h, te_h, rw_h = prob.x_h, prob.gy_h, prob.te_h, prob.rw_h
    ws = prob.ws
    x_e, gy_e, rw_e = ws.x_buffer, ws.d_y_buffer, ws.router_weight_buffer        # host -> symmetric buffers directly
    te_e = torch.empty_like(te_h, device=device)
    res_h = torch.empty(2, dtype=torch.float32).pin_memory()

    def e2e_step():
        x_e.copy_(x_h, non_blocking=True)
        te_e.copy_(te_h, non_blocking=True)
        rw_e.copy_(rw_h, non_blocking=True)
        gy_e.copy_(gy_h, non_blocking=True)
        _, out, grads = prob.step(x_e, te_e, rw_e, gy_e)
        res = torch.stack([out.float().sum(), grads[0].float().sum()])
        res_h.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()     # the caller consumes the result on the host
    for _ in range(2):
        e2e_step()
    e2e_ms = timed(e2e_step, steps)[0] / steps
    h2d = sum(t.numel() * t.element_size() for t in (x_h, te_h, rw_h, gy_h))
    assert _C.check_status() == 0, f"device status word set during the end-to-end steps: {_C.status_detail()}"

    # the same with double-buffered inputs: two workspaces used alternately; step i+1's four inputs cross PCIe on a copy
    # stream straight into the other workspace's symmetric buffers while step i computes (one host->device copy of all
    # four inputs and one device->host read of the checksums per step, as above; no device-side staging copy)
    F = prob.F
    ws2 = F.create_workspace(prob.cfg, prob.group, device=device, num_local_tokens=prob.T, hidden_size=prob.H, topk=prob.K)
    spaces = [ws, ws2]
    te_slots = [te_e, torch.empty_like(te_e)]
    copy_stream = torch.cuda.Stream(device=device)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    pipe = {"i": 0}

    def prefetch(slot):
        w_ = spaces[slot]
        with torch.cuda.stream(copy_stream):     # the slot's last consumer finished two steps ago (each step ends with a synchronize)
            w_.x_buffer.copy_(x_h, non_blocking=True)
            te_slots[slot].copy_(te_h, non_blocking=True)
            w_.router_weight_buffer.copy_(rw_h, non_blocking=True)
            w_.d_y_buffer.copy_(gy_h, non_blocking=True)
            ready[slot].record(copy_stream)

    def e2e_prefetch_step():
        slot = pipe["i"] & 1
        torch.cuda.current_stream().wait_event(ready[slot])
        w_ = spaces[slot]
        _, out, grads = prob.step(w_.x_buffer, te_slots[slot], w_.router_weight_buffer, w_.d_y_buffer, ws=w_)
        prefetch(slot ^ 1)
        res = torch.stack([out.float().sum(), grads[0].float().sum()])
        res_h.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pipe["i"] += 1
    prefetch(0)
    for _ in range(2):
        e2e_prefetch_step()
    e2e_prefetch_ms = timed(e2e_prefetch_step, steps)[0] / steps
    copy_stream.synchronize()
    assert _C.check_status() == 0, f"device status word set during the double-buffered end-to-end steps: {_C.status_detail()}"
    del ws2, spaces
    return {"value": e2e_prefetch_ms, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8,
            "ms_per_step": e2e_prefetch_ms,
            "how": "mok.functional build_schedule + forward + backward; every step's four inputs are copied from pinned host memory "
                   "(double-buffered: step i+1's copies run on a copy stream into a second workspace while step i computes) "
                   "and two checksums are read back to the host",
            "serial": {"value": prob.T * prob.world / (e2e_ms / 1000.0), "ms_per_step": e2e_ms,
                       "note": "the same with the copies on the compute stream before each step"}}


def run_mxfp8_leg(prob, timed, args, _C, ops, sched, real_rows, peak_tf, trace_lines, in_step, rank, device):
    T, H, I, K, E_l, MB = prob.T, prob.H, prob.I, prob.K, prob.E_l, prob.MB
    for _ in range(args.warmup):
        prob.step_mx()
    torch.cuda.synchronize()
    total, per_step = timed(prob.step_mx, args.steps)
    mx_ms = total / args.steps
    mx_f, mx_b = fwd_bwd_split(prob, prob.step_mx, 2)
    assert _C.check_status() == 0, f"device status word set during the MXFP8 steps: {_C.status_detail()}"
    rec = traced_step(_C, prob.step_mx)
    trace_lines += [("mxfp8",) + r for r in rec]
    in_step["mxfp8"] = in_step_summary(rec, "gemm_mxfp8", prob, real_rows, peak_tf)
    mx = {"value": T * prob.world / (mx_ms / 1000.0), "unit": "tokens/s", "ms_per_step": mx_ms,
          "median_ms_per_step": statistics.median(per_step),
          "tflops_per_gpu": prob.flops() / (mx_ms / 1000.0) / 1e12, "fwd_ms": mx_f, "bwd_ms": mx_b,
          "note": "routed experts in block-scaled E4M3 (tcgen05 mxf8f6f4), shared expert BF16; inputs resident in HBM"}
    qg, qu, qd = prob.quantise_weights()
    mx["dominant_kernel"] = time_dominant_kernel_mxfp8(_C, ops, sched, prob.x_d, qg, qu, T, H, I, E_l, MB, 5, 2, device, qd=qd)
    mx["gate_up_launch_alone"] = time_dominant_kernel_mxfp8(_C, ops, sched, prob.x_d, qg, qu, T, H, I, E_l, MB, 5, 2, device)
    prob.q = None
    del qg, qu, qd
    torch.cuda.empty_cache()
    if rank == 0:
        lib = cublaslt_mxfp8_tflops(device)
        if isinstance(lib, tuple):
            mx["cublaslt_mxfp8_tflops"] = {"burst": lib[0], "sustained": lib[1],
                                           "note": "8192^3 torch._scaled_mm with E8M0 block scales, measured in this run"}
            mx["roofline"] = {"bound": "tensor", "kernel": mx["dominant_kernel"]["kernel"], "achieved": mx["dominant_kernel"]["tflops"],
                              "peak": lib[0], "unit": "TFLOP/s", "frac": mx["dominant_kernel"]["tflops"] / lib[0],
                              "peak_source": "cuBLASLt block-scaled E4M3 8192^3 GEMM (torch._scaled_mm), burst of 20 calls, measured in "
                                             "this run: MEASURED_PEAKS.json has no FP8 figure"}
        else:
            mx["cublaslt_mxfp8_tflops"] = {"unavailable": lib}
    return mx


def run_graph_leg(prob, timed, steps, no_mxfp8=False):
    """The step (build_schedule + forward + backward through mok.functional) captured once in a CUDA graph and replayed:
    the library never synchronises the host, joins its side streams inside every call and takes its outputs from
    torch's allocator, so the step is captured as it is.  Host time per step drops to one graph launch."""
    out = {}
    for label, fn in (("bf16", prob.step), ("mxfp8", prob.step_mx)):
        if label == "mxfp8" and no_mxfp8:
            continue
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = fn()
        for _ in range(3):
            graph.replay()
        ms = statistics.median(timed(graph.replay, steps)[1])
        out[label] = {"ms_per_step": ms, "tokens_per_s": prob.T / (ms / 1000.0)}
        del keep, graph
    out["note"] = "one graph launch per step; eager figures are in ms_per_step / mxfp8.ms_per_step"
    return out


def time_dominant_kernel(_C, sched, x, wrg, wru, T, H, I, K, E_l, MB, steps, warmup, device, wrd=None):
    """Times the routed forward GEMM alone, on this step's real schedule: the one persistent launch that computes
    gate/up + SwiGLU and the down projection of every window (mode 4; what the layer runs).  Without `wrd`: the
    gate/up + SwiGLU launch (mode 1) only."""
    tpe = sched.tokens_per_expert
    gob = torch.repeat_interleave(torch.arange(E_l, device=device, dtype=torch.int32), (tpe // 128).to(torch.int64))
    gob = torch.cat([gob, torch.full((MB // 128 - gob.numel(),), -1, dtype=torch.int32, device=device)])
    # the rows' values do not matter for the timing: local tokens repeated, not a peer gather
    x_routed = x.repeat((MB + T - 1) // T, 1)[:MB].contiguous()
    gate, up, hid = (torch.empty(MB, I, dtype=torch.bfloat16, device=device) for _ in range(3))
    y = torch.empty(MB, H, dtype=torch.bfloat16, device=device) if wrd is not None else None
    blk = torch.zeros(MB // 256, dtype=torch.int32, device=device)

    def launch():
        if wrd is None:
            _C.grouped_gemm(1, x_routed, wrg, gate, rows=MB, num_rows=sched.num_tokens, group_of_block=gob, G=E_l, N=I, K=H,
                            B2=wru, D2=up, D3=hid)
        else:
            blk.zero_()
            _C.grouped_gemm(4, x_routed, wrg, gate, rows=MB, num_rows=sched.num_tokens, group_of_block=gob, G=E_l, N=I, K=H,
                            B2=wru, D2=up, D3=hid, B3=wrd, D4=y, N2=H, window_rows=8192, blk_done=blk)
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        launch()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    real_rows = int((sched.peer_rank >= 0).sum().item())
    flops = (4.0 if wrd is None else 6.0) * real_rows * H * I      # 2 (+1) GEMMs x 2 * rows * H * I, padding rows not counted
    padded = int(sched.num_tokens.item())
    return {"ms": ms, "flops_per_launch": flops, "tflops": flops / (ms / 1000.0) / 1e12,
            "rows": real_rows, "padded_rows": padded}


def time_wgrad_kernel(_C, sched, T, H, I, E_l, MB, steps, warmup, device):
    """Times one routed weight-gradient launch alone (dW_down[e] = d_y_e^T * hidden_e, mode 3) on this step's schedule,
    each expert's padding rows left out as in the layer."""
    tpe = sched.tokens_per_expert.to(torch.int64)
    offs = torch.cat([torch.zeros(1, dtype=torch.int64, device=device), tpe.cumsum(0)]).to(torch.int32)
    real = torch.zeros(E_l, dtype=torch.int64, device=device)
    n = int(sched.num_tokens.item())
    seg = torch.repeat_interleave(torch.arange(E_l, device=device), tpe)
    real.index_add_(0, seg, (sched.peer_rank[:n] >= 0).to(torch.int64))
    k_end = (offs[:-1].to(torch.int64) + real).to(torch.int32)
    g = torch.Generator(device=device).manual_seed(5)
    d_y = torch.randn(MB, H, generator=g, device=device).to(torch.bfloat16)
    hid = torch.randn(MB, I, generator=g, device=device).to(torch.bfloat16)
    dW = torch.empty(E_l, H, I, dtype=torch.bfloat16, device=device)

    def launch():
        _C.grouped_gemm(3, d_y, hid, dW, rows=MB, group_offsets=offs, G=E_l, M=H, N=I, group_k_end=k_end)
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        launch()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    flops = 2.0 * float(real.sum().item()) * H * I
    return {"ms": ms, "flops_per_launch": flops, "tflops": flops / (ms / 1000.0) / 1e12}


def time_dominant_kernel_mxfp8(_C, ops, sched, x, qg, qu, T, H, I, E_l, MB, steps, warmup, device, qd=None):
    """Times the routed MXFP8 forward GEMM alone, block-scaled E4M3: with `qd` (the down weights) the one persistent
    launch the layer runs (mode 4: gate|up, SwiGLU and the quantisation of gate, up and hidden in the epilogue, then
    the down projection of the same rows); without, its gate|up part (mode 3)."""
    tpe = sched.tokens_per_expert
    gob = torch.repeat_interleave(torch.arange(E_l, device=device, dtype=torch.int32), (tpe // 128).to(torch.int64))
    gob = torch.cat([gob, torch.full((MB // 128 - gob.numel(),), -1, dtype=torch.int32, device=device)])
    x_routed = x.repeat((MB + T - 1) // T, 1)[:MB].contiguous()
    xq, xs, _, _ = ops.mxfp8_quantize(x_routed, True, False)
    del x_routed
    u8 = dict(dtype=torch.uint8, device=device)
    outs = []
    for _ in range(3):                                   # gate, up, hidden: E4M3 [MB, I] + packed scales
        outs += [torch.empty(MB, I, **u8), torch.empty(MB // 128, I // 128, 32, 16, **u8)]
    outs += [torch.empty(I, MB, **u8), torch.empty(I // 128, MB // 128, 32, 16, **u8)]      # hidden along tokens

    y = torch.empty(MB, H, dtype=torch.bfloat16, device=device) if qd is not None else None
    blk = torch.zeros(MB // 256, dtype=torch.int32, device=device)

    def launch():
        if qd is None:
            _C.grouped_gemm_mxfp8(3, xq, xs, qg[0], qg[1], None, rows=MB, num_rows=sched.num_tokens, group_of_block=gob,
                                  G=E_l, N=I, K=H, B2=qu[0], B2_sc=qu[1], quantised_outputs=outs, t_rows=MB)
        else:
            blk.zero_()
            _C.grouped_gemm_mxfp8(4, xq, xs, qg[0], qg[1], y, rows=MB, num_rows=sched.num_tokens, group_of_block=gob,
                                  G=E_l, N=I, K=H, B2=qu[0], B2_sc=qu[1], quantised_outputs=outs, t_rows=MB,
                                  B3=qd[0], B3_sc=qd[1], N2=H, ldd=H, window_rows=8192, blk_done=blk)
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        launch()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    real_rows = int((sched.peer_rank >= 0).sum().item())
    flops = (4.0 if qd is None else 6.0) * real_rows * H * I
    name = ("grouped_gemm_mxfp8_kernel<gate|up + SwiGLU + quantise>" if qd is None else
            "grouped_gemm_mxfp8_kernel<MODE_FWD> (routed gate|up + SwiGLU + quantise + down, one persistent launch)")
    return {"kernel": name, "ms": ms, "flops_per_launch": flops, "tflops": flops / (ms / 1000.0) / 1e12}


if __name__ == "__main__":
    main()
