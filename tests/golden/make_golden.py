"""Generates the golden vectors in this folder from the REFERENCE's own code.

Run from the repository root, in a container where the reference checkout is
available (its path is given on the command line; it is never needed at test
time):

    python tests/golden/make_golden.py /path/to/delta-feedback-experiment

It imports ``delta_feedback_experiment.pkda.PreconditionedKDA`` from that
checkout, builds a layer of the wanted geometry, overwrites the recurrence
parameters (``A_log``, ``dt_bias``, ``log_precond_center``) with the seeded
values, and calls the reference's ``_portable_recurrence``
(``delta_feedback_experiment/pkda.py:355-410``) with autograd, storing inputs,
outputs, final states and all gradients as float32 ``.npz`` files.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs  # noqa: E402

# name -> (B, T, H, D, distribution, with_state, seed)
CASES = {
    "tiny_unit": (2, 24, 2, 8, "unit", False, 11),
    "tiny_production_state": (1, 37, 3, 16, "production", True, 12),
    "d64_cross_chunk_state": (2, 70, 2, 64, "unit", True, 13),
    "d128_production": (1, 130, 1, 128, "production", False, 14),
    "d128_unit_state": (1, 96, 2, 128, "unit", True, 15),
    "decode_steps": (3, 5, 2, 32, "production", True, 16),
}


def run_reference(ref_root: str, case: tuple) -> dict:
    sys.path.insert(0, ref_root)
    from delta_feedback_experiment.pkda import PreconditionedKDA

    B, T, H, D, dist, with_state, seed = case
    data = make_inputs(B, T, H, D, seed=seed, dist=dist, dtype=torch.float32,
                       with_state=with_state)
    layer = PreconditionedKDA(32, num_heads=H, head_dim=D)
    with torch.no_grad():
        layer.A_log.copy_(data["A_log"])
        layer.dt_bias.copy_(data["dt_bias"])
        layer.log_precond_center.copy_(data["log_atk_scale"])
    leaves = {n: data[n].clone().requires_grad_(True)
              for n in ("q", "k", "v", "g", "g_atk", "beta_atk", "beta")}
    S0 = A0 = None
    if with_state:
        S0 = data["initial_state"].clone().requires_grad_(True)
        A0 = data["initial_A_state"].clone().requires_grad_(True)
    o, S, A = layer._portable_recurrence(
        leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
        leaves["g_atk"], leaves["beta_atk"], S0, A0, True)
    dS = torch.randn(S.shape, generator=torch.Generator().manual_seed(seed + 1000))
    loss = (o * data["do"]).sum() + (S * dS).sum()
    wrt = list(leaves.values()) + [layer.A_log, layer.dt_bias, layer.log_precond_center]
    if with_state:
        wrt += [S0, A0]
    grads = torch.autograd.grad(loss, wrt)
    out = {n: data[n].numpy() for n in INPUT_NAMES}
    out["do"] = data["do"].numpy()
    out["d_final_state"] = dS.numpy()
    out["o"] = o.detach().numpy()
    out["final_state"] = S.detach().numpy()
    out["final_A_state"] = A.detach().numpy()
    names = list(leaves.keys()) + ["A_log", "dt_bias", "log_atk_scale"]
    if with_state:
        out["initial_state"] = data["initial_state"].numpy()
        out["initial_A_state"] = data["initial_A_state"].numpy()
        names += ["initial_state", "initial_A_state"]
    for n, gr in zip(names, grads):
        out["d" + n] = gr.numpy()
    return out


def main() -> None:
    ref_root = sys.argv[1]
    torch.set_num_threads(1)
    for name, case in CASES.items():
        out = run_reference(ref_root, case)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **{k: np.asarray(v, dtype=np.float32) for k, v in out.items()})
        print(name, {k: v.shape for k, v in out.items() if k in ("q", "o", "final_state")},
              os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
