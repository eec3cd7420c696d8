"""The host-memory streaming step equals the plain device call (rows are
independent, so cutting the batch into slices changes nothing per row)."""

import pytest
import torch

from conftest import rel_rms
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("slices,with_state,B", [(2, True, 4), (3, False, 4), (8, True, 4), (8, True, 8),
                                                 ((1, 3, 3, 1), True, 8)])
def test_streamed_step_matches_device_call(slices, with_state, B):
    """Slice counts that divide the batch replay a captured graph per slice (three buffer sets in turn:
    with eight slices every set is used more than once); three slices of four rows take the eager path;
    a plan of unequal slices keeps buffer sets and a captured step per slice size."""
    from delta_feedback_experiment_b200 import chunk_precond_kda
    from delta_feedback_experiment_b200.host_pipeline import HostStep

    T, H, D = 192, 2, 128
    d = make_inputs(B, T, H, D, seed=91, dist="unit", dtype=torch.bfloat16, with_state=with_state)
    host = {n: d[n].pin_memory() for n in INPUT_NAMES}
    if with_state:
        host["initial_state"] = d["initial_state"].pin_memory()
        host["initial_A_state"] = d["initial_A_state"].pin_memory()
    do = d["do"].pin_memory()

    step = HostStep("cuda:0", slices=slices)
    got = step(host, do)
    torch.cuda.synchronize()
    got = {k: v.clone() for k, v in got.items()}
    again = step(host, do)          # buffers are reused: the second call gives the same answer
    torch.cuda.synchronize()
    for k in got:
        assert torch.equal(got[k], again[k]), k
    assert step.h2d_bytes > 0 and step.d2h_bytes > 0

    leaves = [d[n].cuda().requires_grad_(True) for n in INPUT_NAMES]
    kw = dict(zip(INPUT_NAMES, leaves))
    centre = kw.pop("log_atk_scale")
    S0 = d["initial_state"].cuda().requires_grad_(True) if with_state else None
    A0 = d["initial_A_state"].cuda().requires_grad_(True) if with_state else None
    o, _, _ = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=False,
                                log_atk_scale=centre, disable_recompute=True)
    wrt = leaves + ([S0, A0] if with_state else [])
    grads = torch.autograd.grad(o, wrt, d["do"].cuda())
    assert torch.equal(got["o"], o.detach().cpu())
    for n, g in zip(INPUT_NAMES[:7], grads[:7]):
        assert torch.equal(got["d" + n], g.cpu()), n
    for n, g in zip(INPUT_NAMES[7:], grads[7:10]):
        assert rel_rms(got["d" + n], g.float().cpu()) < 1e-5, n
    if with_state:
        assert torch.equal(got["dinitial_state"], grads[10].cpu())
        assert torch.equal(got["dinitial_A_state"], grads[11].cpu())
