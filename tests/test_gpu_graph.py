"""A whole layer step (build_schedule + forward + backward through mok.functional) captured in a CUDA graph and replayed:
the launch-bound regime of small layers.  The step forks to the library's side streams and joins them again inside every
call, allocates its outputs through torch's allocator (graph-private pool under capture) and never synchronises the host,
so it can be captured as it is; replays must give the eager result bit for bit, also after the inputs changed in place."""
import pytest
import torch

from oracle import mok_oracle as O
from tests.gpu_common import init_single_rank_group, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mxfp8", [False, True], ids=["bf16", "mxfp8"])
def test_a_layer_step_replays_from_a_cuda_graph(mxfp8):
    from mok import _C, ops, functional as F
    group = init_single_rank_group()
    E_l, T, H, I, K = 8, 1024, 1024, 512, 2                      # config 1 of the benchmark
    inp = to_dev(O.make_inputs(R=1, T=T, H=H, I=I, E=E_l, K=K, seed=31, routing="router")[0])
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=T * K * 2)
    ws = F.get_workspace(cfg, group, device=torch.device("cuda", 0), num_local_tokens=T, hidden_size=H, topk=K)
    if mxfp8:
        q = [ops.mxfp8_quantize(w, True, True) for w in (inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down)]
        fw = [(a, b) for a, b, _, _ in q]
        bw = [q[0], q[1], (q[2][2], q[2][3])]
    else:
        fw = bw = [inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down]
    shared = (inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down)
    # the step's inputs live in the workspace's buffers (fixed addresses, no staging copies)
    x, rw, gy = ws.x_buffer, ws.router_weight_buffer, ws.d_y_buffer
    x.copy_(inp.x); rw.copy_(inp.router_weights); gy.copy_(inp.grad_output)

    def step():
        sched = F.build_schedule(ws, cfg, inp.top_experts, num_local_experts=E_l)
        out, ctx = F.forward(cfg, ws, sched, x, rw, *shared, *fw)
        grads = F.backward(cfg, ws, sched, ctx, gy, x, rw, *shared, *bw)
        return (out,) + tuple(grads)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                                  # warm-up off the default stream, as capture requires
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for scale in (1.0, 0.5):                                       # replay, then replay on changed inputs
        x.copy_(inp.x * scale); gy.copy_(inp.grad_output * scale)
        graph.replay()
        torch.cuda.synchronize()
        got = [t.clone() for t in captured]
        want = step()
        torch.cuda.synchronize()
        assert _C.check_status() == 0, _C.status_detail()
        for i, (a, b) in enumerate(zip(got, want)):
            assert torch.equal(a, b), f"output {i} of the replay differs from the eager step (input scale {scale})"
