"""Pins the CPU oracle of the two operators next to the recurrence against the
golden vectors the reference itself produced (``tests/golden/make_layer_golden.py``
ran ``PreconditionedKDA._project`` and ``PreconditionedKDA.forward`` on CPU,
``delta_feedback_experiment/pkda.py:197-220,290-316,543-547``)."""

import pytest
import torch

from conftest import assert_close, load_golden
from oracle.pkda_layer_oracle import norm_gate_oracle, qkv_conv_oracle

CONV_CASES = ["layer_conv_small", "layer_conv_d128", "layer_conv_taps3_history", "layer_conv_d64_history"]
GATE_CASES = ["layer_gate_small", "layer_gate_d128", "layer_gate_d64"]


def conv_inputs(g):
    """Rows the fused operator sees: the histories, if any, come first."""
    if "prefix" in g:
        return torch.cat((g["prefix"], g["x"]), dim=1), g["prefix"].shape[1]
    return g["x"], 0


@pytest.mark.parametrize("name", CONV_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_conv_oracle_matches_reference_golden(name, dtype):
    g = load_golden(name)
    rows, skip = conv_inputs(g)
    x = rows.clone().requires_grad_(True)
    w = g["weight"].clone().requires_grad_(True)
    q, k, v = qkv_conv_oracle(x, w, int(g["head_dim"]), int(g["norm_channels"]), float(g["eps"]), dtype)
    for key, val in (("q", q), ("k", k), ("v", v)):
        assert_close(val[:, skip:], g[key], 2e-5, f"{name}:{key}")
    loss = sum((val[:, skip:] * g["d" + key].to(dtype)).sum() for key, val in (("q", q), ("k", k), ("v", v)))
    dx, dw = torch.autograd.grad(loss, [x, w])
    assert_close(dx[:, skip:], g["dx"], 2e-4, f"{name}:dx")
    assert_close(dw, g["dweight"], 2e-4, f"{name}:dweight")
    if skip:
        assert_close(dx[:, :skip], g["dprefix"], 2e-4, f"{name}:dprefix")


@pytest.mark.parametrize("name", GATE_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_norm_gate_oracle_matches_reference_golden(name, dtype):
    g = load_golden(name)
    x = g["x"].clone().requires_grad_(True)
    gate = g["gate"].clone().requires_grad_(True)
    w = g["weight"].clone().requires_grad_(True)
    y, rstd = norm_gate_oracle(x, gate, w, float(g["eps"]), dtype)
    assert_close(y, g["y"], 2e-5, f"{name}:y")
    assert rstd.shape == (x.numel() // x.shape[-1],)
    dx, dg, dw = torch.autograd.grad((y * g["dy"].to(dtype)).sum(), [x, gate, w])
    assert_close(dx, g["dx"], 2e-4, f"{name}:dx")
    assert_close(dg, g["dgate"], 2e-4, f"{name}:dgate")
    assert_close(dw, g["dweight"], 2e-4, f"{name}:dweight")


def test_conv_is_causal_and_row_independent():
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(2, 12, 48, generator=gen)
    w = torch.randn(48, 4, generator=gen)
    base = qkv_conv_oracle(x, w, 8, 32, 1e-6)
    x2 = x.clone()
    x2[0, 7:] += 1.0          # the future of row 0 changes ...
    x2[1] = torch.randn(12, 48, generator=gen)   # ... and all of row 1
    other = qkv_conv_oracle(x2, w, 8, 32, 1e-6)
    for a, b in zip(base, other):
        assert torch.equal(a[0, :7], b[0, :7])


DECODE_CASES = ["layer_decode_small", "layer_decode_d128", "layer_decode_taps2_d64"]


def decode_golden_steps(g):
    """Yields per step (inputs dict, expected dict) of a decode golden file."""
    for t in range(int(g["steps"])):
        ins = {k: g[f"{k}_{t}"] for k in ("qkv", "g", "beta", "g_atk", "beta_atk", "gate")}
        exp = {"out": g[f"out_{t}"], "state": g[f"state_{t}"], "a_state": g[f"a_state_{t}"],
               "conv": [g[f"conv_{t}_{i}"] for i in range(3)]}
        yield ins, exp


@pytest.mark.parametrize("name", DECODE_CASES)
def test_decode_step_oracle_matches_reference_golden(name):
    from oracle.pkda_layer_oracle import decode_step_oracle
    g = load_golden(name)
    state, a_state = g["state0"], g["a_state0"]
    conv = [g[f"conv0_{i}"] for i in range(3)]
    for t, (ins, exp) in enumerate(decode_golden_steps(g)):
        out, state, a_state, conv = decode_step_oracle(
            ins["qkv"], conv, g["conv_weight"], ins["g"], ins["g_atk"], ins["beta_atk"], ins["beta"],
            g["A_log"], g["dt_bias"], g["log_atk_scale"], state, a_state, ins["gate"], g["norm_weight"],
            int(g["head_dim"]), float(g["squash_x"]), float(g["squash_eps"]), float(g["qk_eps"]),
            float(g["norm_eps"]))
        assert_close(out, exp["out"], 2e-5, f"{name}:out{t}")
        assert_close(state, exp["state"], 2e-5, f"{name}:state{t}")
        assert_close(a_state, exp["a_state"], 2e-5, f"{name}:a_state{t}")
        for i in range(3):
            assert torch.equal(conv[i], exp["conv"][i]), f"{name}:conv{t}_{i}"


CONTROL_CASES = ["layer_controls_small", "layer_controls_d128"]


@pytest.mark.parametrize("name", CONTROL_CASES)
def test_controls_oracle_matches_reference_golden(name):
    from oracle.pkda_layer_oracle import controls_oracle
    g = load_golden(name)
    packed = g["packed"].clone().requires_grad_(True)
    A = g["A_log_precond"].clone().requires_grad_(True)
    b = g["dt_bias_precond"].clone().requires_grad_(True)
    outs = controls_oracle(packed, A, b, int(g["hidden"]))
    names = ("decay_hidden", "beta", "g_atk", "beta_atk", "gate_hidden")
    for n, o in zip(names, outs):
        assert_close(o, g[n], 2e-5, f"{name}:{n}")
    loss = sum((o * g["d_" + n]).sum() for n, o in zip(names, outs))
    dp, dA, db = torch.autograd.grad(loss, [packed, A, b])
    assert_close(dp, g["d_packed"], 2e-4, f"{name}:d_packed")
    assert_close(dA, g["dA_log_precond"], 2e-4, f"{name}:dA")
    assert_close(db, g["ddt_bias_precond"], 2e-4, f"{name}:db")
