"""The operators enqueue a fixed sequence of launches on the current stream and
never synchronise, so a forward+backward can be captured into a CUDA graph and
replayed (the reference's benchmark and trainer do exactly that,
``scripts/pkda_bench.py:242-255``)."""

import pytest
import torch

from delta_feedback_experiment_b200 import chunk_precond_kda, pkda_recurrence
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

pytestmark = pytest.mark.gpu


def test_forward_backward_replays_from_a_cuda_graph():
    B, T, H, D = 2, 256, 4, 128
    d = make_inputs(B, T, H, D, seed=5, dist="production", dtype=torch.bfloat16, with_state=True)
    static = {n: d[n].cuda() for n in INPUT_NAMES}
    S0, A0, do = d["initial_state"].cuda(), d["initial_A_state"].cuda(), d["do"].cuda()

    def step():
        leaves = [static[n].detach().requires_grad_(True) for n in INPUT_NAMES]
        s0, a0 = S0.detach().requires_grad_(True), A0.detach().requires_grad_(True)
        kw = dict(zip(INPUT_NAMES, leaves))
        centre = kw.pop("log_atk_scale")
        o, S, A = chunk_precond_kda(**kw, initial_state=s0, initial_A_state=a0, output_final_state=True,
                                    log_atk_scale=centre)
        return (o, S, A) + torch.autograd.grad(o, leaves + [s0, a0], do)

    eager = [t.clone() for t in step()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)
    # new data in the static inputs, same graph
    static["v"].copy_(torch.randn_like(static["v"]))
    graph.replay()
    torch.cuda.synchronize()
    fresh = step()
    for a, b in zip(fresh, captured):
        assert torch.equal(a, b)


def test_custom_op_and_layer_ops_capture():
    from delta_feedback_experiment_b200.layer_ops import pkda_norm_gate, pkda_qkv_conv
    B, T, H, D = 1, 192, 2, 128
    W = H * D
    d = make_inputs(B, T, H, D, seed=6, dist="unit", dtype=torch.bfloat16)
    x = torch.randn(B, T, 3 * W, device="cuda").bfloat16()
    wconv = torch.randn(3 * W, 4, device="cuda") * 0.5
    gate = torch.randn(B, T, H, D, device="cuda").bfloat16()
    wn = torch.ones(D, device="cuda")
    rest = [d[n].cuda() for n in INPUT_NAMES[3:]]

    def step():
        xl, wl = x.detach().requires_grad_(True), wconv.detach().requires_grad_(True)
        q, k, v = pkda_qkv_conv(xl, wl, D, 2 * W, 1e-6)
        sh = (B, T, H, D)
        o, _saved = pkda_recurrence(q.view(sh), k.view(sh), v.view(sh), *rest, D ** -0.5, 1.5, 1e-6, True)
        y, _rstd = pkda_norm_gate(o, gate, wn, 1e-6)
        return (y,) + torch.autograd.grad(y.float().sum(), [xl, wl])

    eager = [t.clone() for t in step()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)
