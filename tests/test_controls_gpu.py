"""GPU parity of the control epilogue (split + sigmoid / softplus forward, packed
gradient in one pass backward) and of the gradient packer, through the C ABI."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from test_layer_oracle import CONTROL_CASES

pytestmark = pytest.mark.gpu
NAMES = ("decay_hidden", "beta", "g_atk", "beta_atk", "gate_hidden")


@pytest.mark.parametrize("name", CONTROL_CASES)
def test_controls_fp32_match_reference_golden(name):
    from delta_feedback_experiment_b200.layer_ops import pkda_controls
    g = load_golden(name)
    packed = g["packed"].cuda().requires_grad_(True)
    A = g["A_log_precond"].cuda().requires_grad_(True)
    b = g["dt_bias_precond"].cuda().requires_grad_(True)
    outs = pkda_controls(packed, A, b, int(g["hidden"]))
    for n, o in zip(NAMES, outs):
        assert_close(o, g[n], 1e-4, f"{name}:{n}")
    assert outs[2].dtype == torch.float32
    loss = sum((o * g["d_" + n].cuda()).sum() for n, o in zip(NAMES, outs))
    dp, dA, db = torch.autograd.grad(loss, [packed, A, b])
    assert_close(dp, g["d_packed"], 1e-4, f"{name}:d_packed")
    assert_close(dA, g["dA_log_precond"], 1e-4, f"{name}:dA")
    assert_close(db, g["ddt_bias_precond"], 1e-4, f"{name}:db")


def test_controls_bf16_match_oracle_and_are_deterministic():
    from delta_feedback_experiment_b200.layer_ops import pkda_controls
    from oracle.pkda_layer_oracle import controls_oracle
    B, T, H, D = 3, 700, 16, 128
    gen = torch.Generator().manual_seed(12)
    packed = torch.randn(B, T, 2 * D + 3 * H, generator=gen).bfloat16()
    A = torch.log(torch.empty(H).uniform_(1, 8, generator=gen))
    b = 0.3 * torch.randn(H, generator=gen)
    cot = [torch.randn(B, T, D, generator=gen).bfloat16(), torch.randn(B, T, H, generator=gen).bfloat16(),
           torch.randn(B, T, H, generator=gen), torch.randn(B, T, H, generator=gen).bfloat16(), None]
    po, Ao, bo = packed.float().requires_grad_(True), A.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = controls_oracle(po, Ao, bo, D)
    rl = sum((o * c.float()).sum() for o, c in zip(ref, cot) if c is not None)
    rdp, rdA, rdb = torch.autograd.grad(rl, [po, Ao, bo])
    runs = []
    for _ in range(2):
        pg, Ag, bg = packed.cuda().requires_grad_(True), A.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
        outs = pkda_controls(pg, Ag, bg, D)
        loss = sum((o.float() * c.cuda().float()).sum() for o, c in zip(outs, cot) if c is not None)
        runs.append((outs, torch.autograd.grad(loss, [pg, Ag, bg])))
    outs, (dp, dA, db) = runs[0]
    for n, o, r in zip(NAMES, outs, ref):
        assert_close(o, r, 2e-2, n)
    assert_close(dp, rdp, 2e-2, "d_packed")
    assert rel_rms(dA, rdA) < 1e-2 and rel_rms(db, rdb) < 1e-2
    assert dp[..., -D:].abs().max() == 0          # no gradient came in for the gate hidden slice
    for a_, b_ in zip(runs[0][1], runs[1][1]):
        assert torch.equal(a_, b_)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_pack_control_gradients_is_cat(dtype):
    from delta_feedback_experiment_b200 import layer_ops  # registers the op
    gen = torch.Generator().manual_seed(4)
    sizes = (128, 16, 16, 16, 128)
    grads = [torch.randn(2, 333, s, generator=gen).to(dtype).cuda() for s in sizes]
    want = torch.cat(grads, dim=-1)
    assert torch.equal(layer_ops.pack_control_gradients(tuple(grads)), want)
    assert torch.equal(torch.ops.delta_feedback.pack_control_gradients(*grads), want)
    with pytest.raises(ValueError):
        layer_ops.pack_control_gradients(tuple(grads[:4]))
