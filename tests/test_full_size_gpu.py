"""Full-size configurations checked through size-independent properties: the packed
variable-length configuration (65,536 tokens, 32 heads) and the long-sequence
configuration.  Sequences (and rows, and heads) are independent, so any sequence
of the big run must equal the same sequence run alone, and one (sequence, head)
slice is compared with the CPU oracle."""

import pytest
import torch

from conftest import assert_close, rel_rms
from delta_feedback_experiment_b200 import chunk_precond_kda
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs, packed_lengths
from oracle.pkda_oracle import pkda_oracle_with_grads

pytestmark = pytest.mark.gpu
ROWS = INPUT_NAMES[:7]


def _run(dev, S0, A0, do, cu=None):
    leaves = {n: dev[n].clone().requires_grad_(True) for n in INPUT_NAMES}
    S0 = S0.clone().requires_grad_(True)
    A0 = A0.clone().requires_grad_(True)
    kw = {n: leaves[n] for n in INPUT_NAMES if n != "log_atk_scale"}
    o, S, A = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=True,
                                log_atk_scale=leaves["log_atk_scale"], cu_seqlens=cu)
    grads = torch.autograd.grad(o, [leaves[n] for n in ROWS] + [S0], do)
    return o, S, A, dict(zip(list(ROWS) + ["S0"], grads))


def test_packed_config_sequences_are_independent_and_match_oracle():
    total, H, D = 65536, 32, 128
    offs = packed_lengths(total, 128, 8192, seed=2)
    N = len(offs) - 1
    d = make_inputs(1, total, H, D, seed=200, dist="unit", dtype=torch.bfloat16, with_state=True, n_states=N)
    dev = {n: d[n].cuda() for n in INPUT_NAMES}
    S0, A0, do = d["initial_state"].cuda(), d["initial_A_state"].cuda(), d["do"].cuda()
    cu = torch.tensor(offs, dtype=torch.int32, device="cuda")
    o, S, A, g = _run(dev, S0, A0, do, cu)
    assert all(torch.isfinite(t.float()).all() for t in (o, S, A, *g.values()))
    # the shortest and one other sequence, each run alone as a dense batch of one
    lens = [offs[i + 1] - offs[i] for i in range(N)]
    picks = sorted(range(N), key=lambda i: lens[i])[:1] + [N // 2]
    for i in picks:
        lo, hi = offs[i], offs[i + 1]
        one = {n: (dev[n][:, lo:hi] if n in ROWS else dev[n]) for n in INPUT_NAMES}
        o1, S1, A1, g1 = _run(one, S0[i:i + 1], A0[i:i + 1], do[:, lo:hi])
        # (every kernel is chosen per chunk or per (sequence, head), never from the size of the batch:
        # a sequence of the packed batch and the same sequence alone take the same path, bit for bit)
        assert torch.equal(o[:, lo:hi], o1), f"sequence {i}: o"
        assert torch.equal(S[i:i + 1], S1), f"sequence {i}: S"
        assert torch.equal(A[i:i + 1], A1)
        for n in ("q", "k", "v", "g", "beta"):
            assert torch.equal(g[n][:, lo:hi], g1[n]), f"sequence {i}: d{n}"
        assert torch.equal(g["S0"][i:i + 1], g1["S0"])
    # one (sequence, head) slice against the oracle (the shortest sequence, head 5)
    i, h = picks[0], 5
    lo, hi = offs[i], offs[i + 1]
    sl = [d[n][:, lo:hi, h:h + 1] for n in ROWS] + [d["A_log"][h:h + 1], d["dt_bias"][h * D:(h + 1) * D],
                                                   d["log_atk_scale"][h:h + 1]]
    ref = pkda_oracle_with_grads(sl, d["do"][:, lo:hi, h:h + 1], initial_state=d["initial_state"][i:i + 1, h:h + 1],
                                 initial_A_state=d["initial_A_state"][i:i + 1, h:h + 1], dtype=torch.float64)
    assert_close(o[:, lo:hi, h:h + 1], ref["o"], 2e-2, "o")
    assert_close(S[i:i + 1, h:h + 1], ref["final_state"], 2e-2, "S")
    for n in ("q", "k", "v"):
        assert_close(g[n][:, lo:hi, h:h + 1], ref["d" + n], 2e-2, "d" + n)
    assert rel_rms(g["g"][:, lo:hi, h:h + 1], ref["dg"]) < 0.015


def test_long_sequence_config_rows_are_independent():
    """Per-GPU shape of the 8-GPU configuration (T = 8192, H = 16): finite, and a row of the big
    batch equals the same row run alone."""
    B, T, H, D = 4, 8192, 16, 128   # four of the sixteen rows: the rows are independent
    d = make_inputs(B, T, H, D, seed=201, dist="unit", dtype=torch.bfloat16, with_state=True)
    dev = {n: d[n].cuda() for n in INPUT_NAMES}
    S0, A0, do = d["initial_state"].cuda(), d["initial_A_state"].cuda(), d["do"].cuda()
    o, S, A, g = _run(dev, S0, A0, do)
    assert all(torch.isfinite(t.float()).all() for t in (o, S, A, *g.values()))
    b = 2
    one = {n: (dev[n][b:b + 1] if n in ROWS else dev[n]) for n in INPUT_NAMES}
    o1, S1, A1, g1 = _run(one, S0[b:b + 1], A0[b:b + 1], do[b:b + 1])
    # no kernel is chosen from the size of the batch: a row alone takes the same path, bit for bit
    assert torch.equal(o[b:b + 1], o1), "o"
    assert torch.equal(S[b:b + 1], S1), "S"
    for n in ("q", "k", "v"):
        assert torch.equal(g[n][b:b + 1], g1[n]), "d" + n
