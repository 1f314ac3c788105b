"""The benchmark's reference arm runs on CPU (the oracle port on host cores): its one JSON line must carry the
keys the measurement contract names, with the reference-arm conventions (impl, zero copy bytes, no GPU launches)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3",
                        "--workload", "c1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["steps"] == 1 and d["warmup"] == 3 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and d["gpu_launches"] == 0


def test_reference_arm_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 0 and not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]


def test_reference_arm_uses_all_host_cores_under_a_launcher_that_pins_one_thread():
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm must not inherit that
    env = dict(os.environ, RANK="0", WORLD_SIZE="2", LOCAL_RANK="0", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                        "--warmup", "3", "--workload", "c1"], capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    sample = d["config"]["sample"]
    assert sample["tokens"] % 512 == 0 and sample["tokens"] >= 512 and sample["hidden"] == 1024 and sample["ep_size"] == 1
    assert d["n_gpus"] == 2


def test_parity_summary_and_byte_model():
    import types
    sys.path.insert(0, ROOT)
    import bench
    from tests.parity_cases import summarise
    good = {"rank": 0, "ok": True, "checks": {"case0_gaussian_bf16": {"status": 0, "schedule_exact": True, "output": [0.1, 1e-3, True]},
                                               "case0_gaussian_mxfp8": {"status": 0, "output": [0.3, 2e-2, True]}}}
    bad = {"rank": 1, "ok": False, "checks": {"case0_gaussian_bf16": {"status": 0, "schedule_exact": False, "output": [0.7, 2e-3, False]}}}
    s = summarise([good])
    assert s["ok"] and s["cases"] == 2 and s["worst"]["output"] == [0.1, 1e-3] and s["worst"]["output_mxfp8"] == [0.3, 2e-2]
    s = summarise([good, bad])
    assert not s["ok"] and s["ranks"] == 2 and s["worst"]["output"][0] == 0.7
    assert set(s["failed"]) == {"rank1/case0_gaussian_bf16/schedule_exact", "rank1/case0_gaussian_bf16/output"}
    prob = types.SimpleNamespace(H=2048, I=1024, T=4096, K=4, flops=lambda: 18.0 * 4096 * 5 * 2048 * 1024)
    m = bench.gate_up_bytes(prob, 20224, 32)
    assert m["total"] == 20224 * 2048 * 2 + 32 * 2 * 1024 * 2048 * 2 + 3 * 20224 * 1024 * 2
    recs = [("gemm_bf16_fwd_routed", 0, 0, 0.0, 1.0), ("dispatch", 0, 1, 0.0, 0.5), ("gemm_bf16_nt", 0, 0, 1.0, 2.0)]
    ins = bench.in_step_summary(recs, "gemm_bf16", prob, 16384, 1000.0)
    assert ins["gemm_launches"] == 2 and ins["gemm_busy_ms"] == 2.0 and ins["fwd_routed_ms"] == 1.0 and ins["step_ms_traced"] == 2.0
    assert abs(ins["fwd_routed_tflops"] - 6.0 * 16384 * 2048 * 1024 / 1e-3 / 1e12) < 1e-6
