"""Helpers shared by the GPU parity tests."""
import os

import numpy as np
import torch
import torch.distributed as dist

from oracle import mok_oracle as O


def init_single_rank_group():
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        torch.cuda.set_device(0)
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    return dist.group.WORLD


def to_dev(inp: O.RankInputs) -> O.RankInputs:
    return O.RankInputs(**{k: getattr(inp, k).cuda() for k in inp.__dataclass_fields__})


def assert_close(name, ref, got, tol):
    mx, rel = O.error_stats(ref.cpu(), got.cpu())
    assert np.isfinite(mx) and np.isfinite(rel), (name, mx, rel)
    assert mx <= tol[0] and rel <= tol[1], f"{name}: max abs {mx:.4e} rel {rel:.4e} exceeds {tol}"
    return mx, rel


# GEMM outputs are compared with an fp32 matmul of the same bf16 operands rounded to bf16:
# the only differences are fp32 summation order and one final rounding.
GEMM_TOL = (0.13, 2e-3)
