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


def groups(rows_per_group):
    """(offsets [G+1], group_of_block [rows/128], rows) as device tensors for ragged expert segments."""
    offs = np.concatenate([[0], np.cumsum(rows_per_group)]).astype(np.int32)
    gob = np.concatenate([np.full(n // 128, g, np.int32) for g, n in enumerate(rows_per_group)] or [np.zeros(0, np.int32)])
    return torch.from_numpy(offs).cuda(), torch.from_numpy(gob).cuda(), int(offs[-1])


def dequantize_gpu(fp8: torch.Tensor, packed_scales: torch.Tensor) -> torch.Tensor:
    """O.dequantize on the device, for operands too large to de-quantise on the host in seconds:
    value * 2^(byte - 127), with the scale byte of (row r, 32-column block kb) of a 128 x 128 tile at
    (r % 32) * 16 + (r // 32) * 4 + kb of the packed [rows/128, cols/128, 32, 16] tensor."""
    shape = fp8.shape
    q = fp8.reshape(-1, shape[-1])
    rb, cb = packed_scales.shape[:2]
    s = packed_scales.reshape(rb, cb, 32, 4, 4).permute(0, 3, 2, 1, 4).reshape(rb * 128, cb * 4)
    scale = torch.ldexp(torch.ones((), device=fp8.device), s.to(torch.int32) - 127)
    return (q.float().reshape(q.shape[0], -1, 32) * scale[:, :, None]).reshape(shape)


def ulp_tol(ref: torch.Tensor, ulps: float = 1.0):
    """Tolerance for two fp32-accumulated results rounded to bf16: `ulps` bf16 steps at the largest magnitude
    (a bf16 step is at most 2^-7 of the value), and 2e-3 on the summed relative error."""
    return (float(ref.float().abs().max()) * 2.0 ** -7 * ulps * 1.01 + 1e-6, 2e-3)
