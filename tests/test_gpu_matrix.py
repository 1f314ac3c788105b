"""Shape / knob sweep of the BF16 layer against the oracle, after the matrix the reference runs
(tests/utils.py:11-44 and tests/test_misc.py:1852-1928 there: local-expert counts, top-k 1-8, seeds,
minimum sizes, minibatch and macrobatch settings, clamped SwiGLU), at sizes the oracle finishes in seconds."""
import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.gpu_common import assert_close
from tests.test_gpu_layer import GRAD_KEYS, run_layer

pytestmark = pytest.mark.gpu

CASES = [
    # T,    H,   I,   E,  K, seed, limit, MB,   mb
    (512, 256, 256, 1, 1, 0, None, None, 256),      # all minimums: one expert, top-1
    (512, 256, 128, 32, 8, 1, None, 12288, 256),    # 32 local experts, top-8, mostly padding
    (512, 512, 256, 16, 4, 2, 4.0, None, 512),      # clamped
    (768, 256, 256, 8, 6, 3, None, None, 256),      # T not a power of two (route bytes stay a multiple of the gather chunk)
    (1024, 256, 256, 4, 2, 4, None, 1024, 256),     # several macrobatches
    (512, 768, 640, 4, 3, 5, 0.0, None, 256),       # limit 0.0 is a valid limit; H, I not powers of two
    (512, 256, 256, 8, 2, 6, None, None, 1024),     # one overlap window
]


@pytest.mark.parametrize("T,H,I,E,K,seed,limit,MB,mb", CASES)
def test_layer_matrix(T, H, I, E, K, seed, limit, MB, mb):
    ranks = O.make_inputs(R=1, T=T, H=H, I=I, E=E, K=K, seed=seed, routing="gaussian")
    need = T * K + E * 256
    factor = max(2, -(-need // (T * K)))
    ref = O.layer_forward_backward(ranks, swiglu_limit=limit, schedule_capacity_factor=factor)[0]
    if MB is None:
        MB = T * K * factor
        MB = -(-MB // mb) * mb
    sched, out, ctx, _, grads, ws = run_layer(ranks[0], E, limit=limit, MB=MB, mb=mb, mult=float(factor))
    np.testing.assert_array_equal(sched.peer_rank.cpu().numpy(), ref["peer_rank"])
    np.testing.assert_array_equal(sched.tokens_per_expert.cpu().numpy(), ref["tokens_per_expert"])
    assert_close("output", ref["output"], out, (0.13, 4e-3))
    for k, got in zip(GRAD_KEYS, grads):
        assert_close(k, ref[k], got, O.BF16_TOLERANCE)
