"""The library's environment switches, each in a process of its own (they are read once per process): the parity cases of
tests/parity_cases.py (BF16 and MXFP8, one and several macrobatches, against the CPU oracle) must hold with everything on
the caller's stream, with single-CTA GEMM tiles, with the register-path epilogue stores, and with the staging rows kept."""
import json
import os
import subprocess
import sys
import tempfile

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("switch", ["MOKB_OVERLAP=0", "MOKB_GEMM_CTAS=1", "MOKB_LINE_STORES=0", "MOKB_KEEP_STAGING_ROWS=1"])
def test_parity_cases_hold_under_every_switch(switch):
    name, value = switch.split("=")
    with tempfile.TemporaryDirectory() as tmp:
        env = dict(os.environ, MOKB_TEST_OUT=tmp, NCCL_NVLS_ENABLE="0", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT="29817")
        env[name] = value
        r = subprocess.run([sys.executable, os.path.join(HERE, "multirank_worker.py")], env=env, capture_output=True, text=True,
                           timeout=280)
        path = os.path.join(tmp, "multirank_rank0.json")
        assert os.path.exists(path), f"no report\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
        report = json.load(open(path))
        assert report["ok"], json.dumps(report, indent=1)
        assert r.returncode == 0, r.stderr[-3000:]
