"""The environment the reference runs its operators in (``delta_feedback_experiment/model.py:925-935``,
``fla_ops.py:433-437, 549-556``): the three custom operators of the layer inside one
``torch.compile(fullgraph=True)`` graph, under non-reentrant activation checkpointing with a
bf16-autocast forward and a backward outside autocast, and ``torch.library.opcheck`` on every
registered operator.  Gradients must equal the eager ones bit for bit (same kernels, fixed
reduction orders)."""

import pytest
import torch
from torch.utils.checkpoint import checkpoint

from delta_feedback_experiment_b200 import pkda_recurrence
from delta_feedback_experiment_b200.layer_ops import (_pack_control_gradients_op, pkda_norm_gate,
                                                     pkda_qkv_conv)

pytestmark = pytest.mark.gpu
B, T, H, D = 2, 130, 2, 128
W = H * D


def _block(x, wconv, g, g_atk, beta_atk, beta, A_log, dt_bias, centre, gate, wnorm):
    q, k, v = pkda_qkv_conv(x, wconv, D, 2 * W, 1e-6)
    q, k, v = (t.view(B, T, H, D) for t in (q, k, v))
    o, _saved = pkda_recurrence(q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, centre,
                                D ** -0.5, 1.5, 1e-6, True)
    y, _rstd = pkda_norm_gate(o, gate, wnorm, 1e-6)
    return y


def _inputs(seed=0):
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen)
    bf = torch.bfloat16
    t = [
        rn(B, T, 3 * W).to(bf), rn(3 * W, 4) * 0.5, rn(B, T, H, D).to(bf),
        -torch.nn.functional.softplus(rn(B, T, H)), torch.sigmoid(rn(B, T, H)).to(bf),
        torch.sigmoid(rn(B, T, H)).to(bf), torch.zeros(H), rn(H * D) * 0.1, torch.full((H,), -0.2),
        rn(B, T, H, D).to(bf), 1 + 0.1 * rn(D),
    ]
    return [x.cuda().requires_grad_(True) for x in t], rn(B, T, H, D).to(bf).cuda()


def _grads(fn, autocast=False):
    leaves, dy = _inputs()
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
        y = fn(*leaves)
    return [y] + list(torch.autograd.grad(y, leaves, dy))  # the backward runs outside autocast


def test_fullgraph_compile_matches_eager():
    eager = _grads(_block)
    compiled = torch.compile(_block, fullgraph=True, dynamic=False, backend="aot_eager")
    got = _grads(compiled)
    for a, b in zip(got, eager):
        assert a.dtype == b.dtype and torch.equal(a, b)


def test_nonreentrant_checkpoint_under_autocast_matches_eager():
    eager = _grads(_block)
    got = _grads(lambda *a: checkpoint(_block, *a, use_reentrant=False), autocast=True)
    for a, b in zip(got, eager):
        assert a.dtype == b.dtype and torch.equal(a, b)


def test_opcheck_registered_operators():
    checks = ("test_schema", "test_autograd_registration", "test_faketensor")
    leaves, _ = _inputs(3)
    x, wconv, g, g_atk, beta_atk, beta, A_log, dt_bias, centre, gate, wnorm = leaves
    torch.library.opcheck(pkda_qkv_conv, (x, wconv, D, 2 * W, 1e-6), test_utils=checks)
    with torch.no_grad():
        q, k, v = (t.view(B, T, H, D) for t in pkda_qkv_conv(x, wconv, D, 2 * W, 1e-6))
    q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    for lean in (True, False):
        torch.library.opcheck(
            pkda_recurrence, (q, k, v, g, g_atk, beta_atk, beta, A_log, dt_bias, centre,
                              D ** -0.5, 1.5, 1e-6, lean), test_utils=checks)
    torch.library.opcheck(pkda_norm_gate, (q, gate, wnorm, 1e-6), test_utils=checks)
    parts = [torch.randn(B, T, n, device="cuda", dtype=torch.bfloat16) for n in (16, H, H, H, 16)]
    torch.library.opcheck(_pack_control_gradients_op, tuple(parts), test_utils=checks)
