"""GPU parity of both grouped GEMMs at the shapes the benchmark runs (hidden 7168 / 5120 / 4096, expert
width 2048 / 1408 / 1536): long contractions (up to 112 shared-memory stages per tile, about 19 trips round
the ring), several tiles per CTA pair so that both accumulator phases wrap, ragged groups with an empty one,
and column counts that are not multiples of 256.  Reference: fp32 matmul on the device with TF32 off, of the
bf16 operands (BF16) or of the de-quantised operands (MXFP8), per group."""
import pytest
import torch

from tests.gpu_common import assert_close, dequantize_gpu, groups, ulp_tol

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fp32_matmul_exact():
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = old
    torch.cuda.empty_cache()


def randn(*shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def pairs_walk_three_tiles(tiles):
    from mok import _C
    assert tiles >= 3 * (_C.lib.mokb_sm_count() // 2), "case too small: every CTA pair must walk at least three tiles"


# (rows per group, H, I): config 2, config 5 (I = 11 * 128), config 4
FWD_SHAPES = [([1024, 0, 2560, 512], 7168, 2048), ([2048, 0, 3072, 512], 5120, 1408), ([512, 4608, 0, 256], 4096, 1536)]
DOWN_SHAPES = [([1024, 0, 2560, 512], 7168, 2048), ([2560, 0, 1024, 512], 5120, 1408), ([512, 3328, 0, 256], 4096, 1536)]
DGRAD_SHAPES = [([2048, 0, 4608, 512], 7168, 2048), ([3072, 0, 5888, 512], 5120, 1408), ([512, 7936, 0, 1024], 4096, 1536)]


@pytest.mark.parametrize("rows_per_group,H,I", FWD_SHAPES, ids=["c2", "c5", "c4"])
def test_bf16_gate_up_swiglu_at_benchmark_shapes(rows_per_group, H, I):
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    pairs_walk_three_tiles((rows // 256) * (I // 128))
    A = randn(rows, H, seed=1)
    Wg, Wu = randn(G_, I, H, seed=2, scale=0.02), randn(G_, I, H, seed=3, scale=0.02)
    gate, up, hid = (torch.empty(rows, I, dtype=torch.bfloat16, device="cuda") for _ in range(3))
    _C.grouped_gemm(1, A, Wg, gate, group_of_block=gob, G=G_, N=I, K=H, B2=Wu, D2=up, D3=hid)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        rg = A[s:e].float() @ Wg[gi].float().T
        ru = A[s:e].float() @ Wu[gi].float().T
        assert_close("gate", rg.to(torch.bfloat16), gate[s:e], ulp_tol(rg))
        assert_close("up", ru.to(torch.bfloat16), up[s:e], ulp_tol(ru))
        g32, u32 = gate[s:e].float(), up[s:e].float()
        assert_close("hidden", (torch.nn.functional.silu(g32) * u32).to(torch.bfloat16), hid[s:e], (0.05, 2e-3))


@pytest.mark.parametrize("rows_per_group,H,I", DOWN_SHAPES, ids=["c2", "c5", "c4"])
def test_bf16_down_at_benchmark_shapes(rows_per_group, H, I):
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    pairs_walk_three_tiles((rows // 256) * (H // 256))
    A = randn(rows, I, seed=4)
    W = randn(G_, H, I, seed=5, scale=0.02)
    D = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(0, A, W, D, group_of_block=gob, G=G_, N=H, K=I)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s < e:
            ref = A[s:e].float() @ W[gi].float().T
            assert_close(f"down group {gi}", ref.to(torch.bfloat16), D[s:e], ulp_tol(ref))


@pytest.mark.parametrize("rows_per_group,H,I", DGRAD_SHAPES, ids=["c2", "c5", "c4"])
def test_bf16_input_gradients_at_benchmark_shapes(rows_per_group, H, I):
    """d_hidden = d_y * W_down (contraction over H) and d_x = d_gate * W_gate + d_up * W_up (two operand pairs, I each)."""
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    pairs_walk_three_tiles((rows // 256) * ((I + 255) // 256))
    dy = randn(rows, H, seed=6)
    Wd = randn(G_, H, I, seed=7, scale=0.02)
    dh = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(2, dy, Wd, dh, group_of_block=gob, G=G_, N=I, K=H)
    dg, du = randn(rows, I, seed=8), randn(rows, I, seed=9)
    Wg, Wu = randn(G_, I, H, seed=10, scale=0.02), randn(G_, I, H, seed=11, scale=0.02)
    dx = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(2, dg, Wg, dx, group_of_block=gob, G=G_, N=H, K=I, A2=du, B2=Wu)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        ref = dy[s:e].float() @ Wd[gi].float()
        assert_close(f"d_hidden group {gi}", ref.to(torch.bfloat16), dh[s:e], ulp_tol(ref))
        ref = dg[s:e].float() @ Wg[gi].float() + du[s:e].float() @ Wu[gi].float()
        assert_close(f"d_x group {gi}", ref.to(torch.bfloat16), dx[s:e], ulp_tol(ref, 2.0))


@pytest.mark.parametrize("rows_per_group,H,I", [([1024, 0, 2560], 7168, 2048), ([2048, 0, 512, 1536], 5120, 1408),
                                                ([512, 3584, 0], 4096, 1536)], ids=["c2", "c5", "c4"])
def test_bf16_weight_gradients_at_benchmark_shapes(rows_per_group, H, I):
    """dW_down[g] = d_y_g^T * hidden_g ([H, I]) and dW_gate[g] = d_gate_g^T * x_g ([I, H])."""
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    pairs_walk_three_tiles(G_ * (H // 256) * ((I + 255) // 256))
    dy, hid = randn(rows, H, seed=12), randn(rows, I, seed=13, scale=0.25)
    dWd = torch.full((G_, H, I), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(3, dy, hid, dWd, group_offsets=offs, G=G_, M=H, N=I)
    dg, x = randn(rows, I, seed=14, scale=0.25), randn(rows, H, seed=15)
    dWg = torch.full((G_, I, H), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm(3, dg, x, dWg, group_offsets=offs, G=G_, M=I, N=H)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            assert torch.all(dWd[gi] == 0) and torch.all(dWg[gi] == 0)
            continue
        ref = dy[s:e].float().T @ hid[s:e].float()
        assert_close(f"dW_down group {gi}", ref.to(torch.bfloat16), dWd[gi], ulp_tol(ref))
        ref = dg[s:e].float().T @ x[s:e].float()
        assert_close(f"dW_gate group {gi}", ref.to(torch.bfloat16), dWg[gi], ulp_tol(ref))


# ------------------------------------------------------------------ MXFP8
def quant(x):
    """bf16 [.., R, C] on the device -> (E4M3, packed scales, de-quantised fp32), blocks along the last axis
    (the device quantiser is byte-exact against the oracle: tests/test_gpu_ops.py)."""
    from mok import ops
    q, s, _, _ = ops.mxfp8_quantize(x, True, False)
    return q, s, dequantize_gpu(q.reshape(-1, x.shape[-1]), s).reshape(x.shape)


@pytest.mark.parametrize("rows_per_group,H,I", DOWN_SHAPES, ids=["c2", "c5", "c4"])
def test_mxfp8_down_and_dual_input_gradient_at_benchmark_shapes(rows_per_group, H, I):
    """Mode 0 twice: y = hidden * W_down^T (contraction over I) and, with a second operand pair,
    d_x = d_gate * Wg^T' + d_up * Wu^T' with the weights pre-transposed to [E, H, I]."""
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    Aq, As, Ad = quant(randn(rows, I, seed=21))
    Wq, Ws, Wd = quant(randn(G_, H, I, seed=22, scale=0.02))
    A2q, A2s, A2d = quant(randn(rows, I, seed=23))
    W2q, W2s, W2d = quant(randn(G_, H, I, seed=24, scale=0.02))
    D = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    D2 = torch.empty(rows, H, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(0, Aq, As, Wq, Ws, D, group_of_block=gob, G=G_, N=H, K=I)
    _C.grouped_gemm_mxfp8(0, Aq, As, Wq, Ws, D2, group_of_block=gob, G=G_, N=H, K=I, A2=A2q, A2_sc=A2s, B2=W2q, B2_sc=W2s)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        ref = Ad[s:e] @ Wd[gi].T
        assert_close(f"down group {gi}", ref.to(torch.bfloat16), D[s:e], ulp_tol(ref))
        ref = ref + A2d[s:e] @ W2d[gi].T
        assert_close(f"dual group {gi}", ref.to(torch.bfloat16), D2[s:e], ulp_tol(ref, 2.0))


@pytest.mark.parametrize("rows_per_group,H,I", DGRAD_SHAPES[:1] + FWD_SHAPES[1:], ids=["c2", "c5", "c4"])
def test_mxfp8_long_contraction_at_benchmark_shapes(rows_per_group, H, I):
    """Mode 0 with the contraction over H (d_hidden = d_y * W_down^T', 56 / 40 / 32 stages of 128 bytes per tile) and
    mode 1 (gate and up in one pass) on the same operands."""
    from mok import _C
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    Aq, As, Ad = quant(randn(rows, H, seed=25))
    Wq, Ws, Wd = quant(randn(G_, I, H, seed=26, scale=0.02))
    W2q, W2s, W2d = quant(randn(G_, I, H, seed=27, scale=0.02))
    D = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    G1 = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    U1 = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(0, Aq, As, Wq, Ws, D, group_of_block=gob, G=G_, N=I, K=H)
    _C.grouped_gemm_mxfp8(1, Aq, As, Wq, Ws, G1, group_of_block=gob, G=G_, N=I, K=H, B2=W2q, B2_sc=W2s, D2=U1)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if s == e:
            continue
        ref = Ad[s:e] @ Wd[gi].T
        assert_close(f"group {gi}", ref.to(torch.bfloat16), D[s:e], ulp_tol(ref))
        assert_close(f"gate group {gi}", ref.to(torch.bfloat16), G1[s:e], ulp_tol(ref))
        ref = Ad[s:e] @ W2d[gi].T
        assert_close(f"up group {gi}", ref.to(torch.bfloat16), U1[s:e], ulp_tol(ref))


@pytest.mark.parametrize("rows_per_group,H,I", FWD_SHAPES, ids=["c2", "c5", "c4"])
def test_mxfp8_fused_gate_up_swiglu_quantise_at_benchmark_shapes(rows_per_group, H, I):
    """Mode 3 against mode 1 + the quantiser: gate and up byte-exact, hidden within one E4M3 step."""
    from mok import _C, ops
    offs, gob, rows = groups(rows_per_group)
    G_ = len(rows_per_group)
    Aq, As, _ = quant(randn(rows, H, seed=28))
    Gq, Gs, _ = quant(randn(G_, I, H, seed=29, scale=0.02))
    Uq, Us, _ = quant(randn(G_, I, H, seed=30, scale=0.02))
    gate = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    up = torch.empty(rows, I, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(1, Aq, As, Gq, Gs, gate, group_of_block=gob, G=G_, N=I, K=H, B2=Uq, B2_sc=Us, D2=up)
    u8 = dict(dtype=torch.uint8, device="cuda")
    sc = lambda r, c: torch.zeros(r // 128, c // 128, 32, 16, **u8)
    outs = [torch.zeros(rows, I, **u8), sc(rows, I), torch.zeros(rows, I, **u8), sc(rows, I),
            torch.zeros(rows, I, **u8), sc(rows, I), torch.zeros(I, rows, **u8), sc(I, rows)]
    _C.grouped_gemm_mxfp8(3, Aq, As, Gq, Gs, None, group_of_block=gob, G=G_, N=I, K=H, B2=Uq, B2_sc=Us,
                          quantised_outputs=outs, t_rows=rows)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    gq, gs, _, _ = ops.mxfp8_quantize(gate, True, False)
    uq, us, _, _ = ops.mxfp8_quantize(up, True, False)
    assert torch.equal(outs[0], gq.view(torch.uint8)) and torch.equal(outs[1], gs)
    assert torch.equal(outs[2], uq.view(torch.uint8)) and torch.equal(outs[3], us)
    hidden = _C.swiglu_fwd(gate, up, None)
    hq, hs, hqt, hst = ops.mxfp8_quantize(hidden, True, True)
    f8 = torch.float8_e4m3fn
    for name, got_q, got_s, ref_q, ref_s in (("hidden", outs[4], outs[5], hq, hs), ("hidden^T", outs[6], outs[7], hqt, hst)):
        assert (got_q == ref_q.view(torch.uint8)).float().mean().item() > 0.995, name
        assert_close(name, dequantize_gpu(ref_q, ref_s), dequantize_gpu(got_q.view(f8), got_s), (0.05, 2e-3))


@pytest.mark.parametrize("cols_per_group,H,I", [([1024, 0, 2560], 7168, 2048), ([2048, 0, 512, 1536], 5120, 1408),
                                                ([512, 3584, 0], 4096, 1536)], ids=["c2", "c5", "c4"])
def test_mxfp8_weight_gradients_at_benchmark_shapes(cols_per_group, H, I):
    """Mode 2: dW_down[g] = d_y^T[:, cols_g] * hidden^T[:, cols_g]^T, both operands quantised along tokens."""
    from mok import _C
    offs, gob, cols = groups(cols_per_group)
    G_ = len(cols_per_group)
    Aq, As, Ad = quant(randn(H, cols, seed=31))
    Bq, Bs, Bd = quant(randn(I, cols, seed=32, scale=0.25))
    D = torch.full((G_, H, I), 5.0, dtype=torch.bfloat16, device="cuda")
    _C.grouped_gemm_mxfp8(2, Aq, As, Bq, Bs, D, group_offsets=offs, G=G_, M=H, N=I)
    torch.cuda.synchronize()
    assert _C.check_status() == 0
    o = offs.cpu().numpy()
    for gi in range(G_):
        s, e = int(o[gi]), int(o[gi + 1])
        if e == s:
            assert torch.all(D[gi] == 0)
            continue
        ref = Ad[:, s:e] @ Bd[:, s:e].T
        assert_close(f"wgrad {gi}", ref.to(torch.bfloat16), D[gi], ulp_tol(ref))
