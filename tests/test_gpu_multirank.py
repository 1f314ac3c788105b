"""Expert parallelism over real GPUs (2, 4 and 8 when present): launches tests/multirank_worker.py under
torch.distributed.run and checks every rank's report.  Skipped on a single-GPU machine."""
import json
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_layer_over_peer_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        env = dict(os.environ, MOKB_TEST_OUT=tmp, NCCL_NVLS_ENABLE="0")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(29800 + world), os.path.join(HERE, "multirank_worker.py")]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
        reports = []
        for rank in range(world):
            path = os.path.join(tmp, f"multirank_rank{rank}.json")
            assert os.path.exists(path), f"rank {rank} wrote no report\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
            reports.append(json.load(open(path)))
        assert all(rep["ok"] for rep in reports), json.dumps(reports, indent=1)
        assert r.returncode == 0, r.stderr[-3000:]
