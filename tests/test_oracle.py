"""Pins the CPU oracle against the golden vectors the reference itself produced
(``tests/golden/make_golden.py`` ran ``PreconditionedKDA._portable_recurrence``,
``delta_feedback_experiment/pkda.py:355-410``)."""

import pytest
import torch

from conftest import assert_close, load_golden
from oracle.pkda_oracle import (INPUT_NAMES, pkda_oracle_with_grads,
                                pkda_packed_oracle, pkda_recurrent_oracle)

CASES = ["tiny_unit", "tiny_production_state", "d64_cross_chunk_state",
         "d128_production", "d128_unit_state", "decode_steps"]


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_oracle_matches_reference_golden(name, dtype):
    g = load_golden(name)
    res = pkda_oracle_with_grads(
        [g[n] for n in INPUT_NAMES], g["do"],
        initial_state=g.get("initial_state"), initial_A_state=g.get("initial_A_state"),
        d_final_state=g["d_final_state"], dtype=dtype)
    # fp32 reference vs fp32/fp64 restatement: only summation order differs.
    for key in ("o", "final_state", "final_A_state"):
        assert_close(res[key], g[key], 2e-5, f"{name}:{key}")
    for n in INPUT_NAMES:
        assert_close(res["d" + n], g["d" + n], 2e-4, f"{name}:d{n}")
    if "initial_state" in g:
        assert_close(res["dinitial_state"], g["dinitial_state"], 2e-4, "dS0")
        assert_close(res["dinitial_A_state"], g["dinitial_A_state"], 2e-4, "dA0")


def test_state_carry_equals_full_recompute():
    """Prefill then token-by-token decode equals one pass (the reference pins the
    same property through its cache test, ``tests/test_model.py:467-508``)."""
    g = load_golden("tiny_production_state")
    ins = [g[n] for n in INPUT_NAMES]
    full = pkda_recurrent_oracle(*ins, initial_state=g["initial_state"],
                                 initial_A_state=g["initial_A_state"])
    S, A = g["initial_state"], g["initial_A_state"]
    outs = []
    for lo, hi in [(0, 3)] + [(t, t + 1) for t in range(3, ins[0].shape[1])]:
        part = [t[:, lo:hi] for t in ins[:7]] + ins[7:]
        o, S, A = pkda_recurrent_oracle(*part, initial_state=S, initial_A_state=A)
        outs.append(o)
    assert_close(torch.cat(outs, 1), full[0], 1e-5, "o")
    assert_close(S, full[1], 1e-5, "S")
    assert_close(A, full[2], 1e-5, "A")


def test_packed_equals_per_row():
    """Rows are independent (``tests/test_mtp.py:267-283``): packing two rows
    end to end with ``cu_seqlens`` reproduces the batched result."""
    g = load_golden("tiny_unit")
    ins = [g[n] for n in INPUT_NAMES]
    B, T = ins[0].shape[:2]
    packed = [t.reshape(1, B * T, *t.shape[2:]) for t in ins[:7]] + ins[7:]
    o, S, A = pkda_packed_oracle(*packed, cu_seqlens=[0, T, 2 * T])
    assert_close(o.reshape(B, T, *o.shape[2:]), g["o"], 2e-5, "o")
    assert_close(S, g["final_state"], 2e-5, "S")
    assert_close(A, g["final_A_state"], 2e-5, "A")
