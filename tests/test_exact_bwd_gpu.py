"""GPU parity of the exact (fp32) backward against the reference's own gradients
(golden vectors), at the fp32 tolerance, for every head width; and as an
independent on-device check of the chunked bf16 backward at a size the CPU oracle
cannot reach."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from delta_feedback_experiment_b200 import chunk_precond_kda, ops, pkda_recurrence
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_oracle_with_grads

pytestmark = pytest.mark.gpu
CASES = ["tiny_unit", "tiny_production_state", "d64_cross_chunk_state", "d128_production",
         "d128_unit_state", "decode_steps"]


def run_exact(g, dS=None, cu=None):
    leaves = {n: g[n].cuda().requires_grad_(True) for n in INPUT_NAMES}
    ws = "initial_state" in g
    S0 = g["initial_state"].cuda().requires_grad_(True) if ws else None
    A0 = g["initial_A_state"].cuda().requires_grad_(True) if ws else None
    o, S, A = chunk_precond_kda(
        q=leaves["q"], k=leaves["k"], v=leaves["v"], g=leaves["g"], g_atk=leaves["g_atk"],
        beta_atk=leaves["beta_atk"], beta=leaves["beta"], A_log=leaves["A_log"],
        dt_bias=leaves["dt_bias"], initial_state=S0, initial_A_state=A0, output_final_state=True,
        log_atk_scale=leaves["log_atk_scale"],
        cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda"))
    loss = (o * g["do"].cuda()).sum()
    if dS is not None:
        loss = loss + (S * dS.cuda()).sum()
    wrt = list(leaves.values()) + ([S0, A0] if ws else [])
    grads = torch.autograd.grad(loss, wrt)
    out = {"d" + n: x for n, x in zip(INPUT_NAMES, grads)}
    if ws:
        out["dinitial_state"], out["dinitial_A_state"] = grads[10], grads[11]
    return out


@pytest.mark.parametrize("name", CASES)
def test_fp32_gradients_match_reference_golden(name):
    g = load_golden(name)
    res = run_exact(g, dS=g["d_final_state"])
    # Both sides are fp32 (the golden gradients come from the reference's own fp32
    # autograd), so each carries rounding noise: 1e-4 elementwise for the gradients of
    # q, k, v, beta and the states; the gate / preconditioner gradients are long sums with
    # cancellation (strong-decay cases especially) and get 1e-3 elementwise plus a
    # relative-RMS bound of 3e-4.
    for n in INPUT_NAMES:
        tight = n in ("q", "k", "v", "beta")
        assert_close(res["d" + n], g["d" + n], 1e-4 if tight else 1e-3, f"{name}:d{n}")
        if n not in ("A_log", "dt_bias", "log_atk_scale"):  # per-head sums are a handful of numbers
            assert rel_rms(res["d" + n], g["d" + n]) < 3e-4, (name, n)
    if "initial_state" in g:
        assert_close(res["dinitial_state"], g["dinitial_state"], 1e-4, "dS0")
        assert_close(res["dinitial_A_state"], g["dinitial_A_state"], 1e-3, "dA0")


def test_fp32_packed_gradients():
    lens = [5, 70, 1, 33]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    d = make_inputs(1, offs[-1], 2, 32, seed=9, dist="production", dtype=torch.float32,
                    with_state=True, n_states=len(lens))
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], cu_seqlens=offs,
                                 dtype=torch.float64)
    res = run_exact(d, cu=offs)
    for n in INPUT_NAMES:
        assert_close(res["d" + n], ref["d" + n], 5e-4, "d" + n)


def test_custom_op_fp32_all_ten_gradients():
    d = make_inputs(2, 100, 2, 64, seed=11, dist="unit", dtype=torch.float32)
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"], dtype=torch.float64)
    leaves = [d[n].cuda().requires_grad_(True) for n in INPUT_NAMES]
    o, _ = pkda_recurrence(*leaves, 64 ** -0.5, 1.5, 1e-6, True)
    grads = torch.autograd.grad(o, leaves, d["do"].cuda())
    assert_close(o, ref["o"], 1e-4, "o")
    for n, gr in zip(INPUT_NAMES, grads):
        assert_close(gr, ref["d" + n], 5e-4, "d" + n)


def test_chunked_bf16_backward_against_exact_kernel_at_full_length():
    """T = 4096 (64 chunks), d = 128: the chunked bf16 gradients against the exact
    kernel on the same bf16 inputs -- a full-length check the CPU oracle cannot do."""
    B, T, H, D = 1, 4096, 4, 128
    d = make_inputs(B, T, H, D, seed=13, dist="unit", dtype=torch.bfloat16, with_state=True)
    t = [d[n].cuda() for n in INPUT_NAMES]
    S0, A0, do = d["initial_state"].cuda(), d["initial_A_state"].cuda(), d["do"].cuda()
    exact, eS0, _ = ops.recurrent_backward(*t, D ** -0.5, 1.5, 1e-6, do, S0, A0, None, None, True)
    o, _, _, saved = ops.chunk_forward(*t, D ** -0.5, 1.5, 1e-6, S0, A0, None, False)
    chunk, cS0, _ = ops.chunk_backward(*t, D ** -0.5, 1.5, 1e-6, saved, do, S0, A0, None, None, False, True)
    # per-token tensors: the reference benchmark's limits; the three per-head parameter
    # gradients are 4-element vectors here, each a cancelling sum over 4096 x 128 terms: 0.05
    limits = (0.007, 0.008, 0.007, 0.015, 0.015, 0.015, 0.015, 0.05, 0.05, 0.05)
    for n, a, e, lim in zip(INPUT_NAMES, chunk, exact, limits):
        assert rel_rms(a, e) < lim, f"d{n}: {rel_rms(a, e):.3e}"
    assert rel_rms(cS0, eS0) < 0.01
