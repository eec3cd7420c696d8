"""Run-to-run determinism where CTAs hand data to one another inside a kernel.

With 32 or more (row, head) units the forward intra-chunk kernel carries the preconditioner
state from the item of one chunk to the item of the next (counters in global memory,
release / acquire), the work lists are filled through atomic cursors and the state scans
hand tiles between warp groups.  None of that may show in the results: two runs of the same
problem must agree bit for bit, every status word must stay 0, and the chained forward must
give the bits of the path that computes the same state with two small kernels in front
(fewer than 32 units: the same rows run alone)."""

import pytest
import torch

from delta_feedback_experiment_b200 import chunk_precond_kda, ops
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

pytestmark = pytest.mark.gpu
D = 128


def _run(d, dS):
    leaves = {n: d[n].cuda().clone().requires_grad_(True) for n in INPUT_NAMES}
    S0 = d["initial_state"].cuda().clone().requires_grad_(True)
    A0 = d["initial_A_state"].cuda().clone().requires_grad_(True)
    kw = {n: leaves[n] for n in INPUT_NAMES if n != "log_atk_scale"}
    o, S, A = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=True,
                                log_atk_scale=leaves["log_atk_scale"])
    g = torch.autograd.grad([o, S], [leaves[n] for n in INPUT_NAMES] + [S0, A0], [d["do"].cuda(), dS.cuda()])
    assert ops.last_device_status() == 0 and ops.last_backward_status() == 0
    return [o, S, A, *g]


@pytest.mark.parametrize("B,H,T,dist", [(8, 16, 1000, "unit"), (4, 8, 2048, "unit"), (16, 2, 511, "production"),
                                        (9, 4, 200, "unit"), (2, 16, 65, "production")])
def test_two_runs_agree_bit_for_bit(B, H, T, dist):
    d = make_inputs(B, T, H, D, seed=7 * B + H, dist=dist, dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(3)) * 0.1
    first = _run(d, dS)
    for _ in range(2):
        again = _run(d, dS)
        for x, y in zip(first, again):
            assert torch.equal(x, y)
            assert torch.isfinite(x.float()).all()


def test_chained_state_equals_the_unchained_path():
    """8 rows x 8 heads = 64 units: the forward chains the preconditioner state inside the intra kernel.
    Two rows alone are 16 units: two small kernels compute the same state in front.  Per-row results
    (the final preconditioner state among them) must be the same bits."""
    B, H, T = 8, 8, 777
    d = make_inputs(B, T, H, D, seed=29, dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(4)) * 0.1
    whole = _run(d, dS)
    two = {k: (v[2:4] if torch.is_tensor(v) and v.dim() >= 3 and v.shape[0] == B else v) for k, v in d.items()}
    part = _run(two, dS[2:4])
    names = ["o", "S", "A"] + ["d" + n for n in INPUT_NAMES] + ["dS0", "dA0"]
    for name, x, y in zip(names, whole, part):
        if name in ("dA_log", "ddt_bias", "dlog_atk_scale"):
            continue  # sums over rows
        assert torch.equal(x[2:4], y), name
