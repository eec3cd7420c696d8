"""The two timed chunked configurations at their real shapes against the CPU oracle:
B=8, T=4096, H=16 (one GPU) and B=16, T=8192, H=16 (the per-GPU shape of the eight-GPU
run).  The whole problem runs on the GPU, through the tcgen05 / tensor-memory kernels that
the benchmark times, and one (row, head)
slice is compared with the float64 oracle: output, both final states, the seven per-token
gradients and both initial-state gradients.  The three per-head parameter gradients are sums
over all rows, so they are checked on a GPU run of the slice alone."""

import pytest
import torch

from conftest import assert_close, rel_rms
from delta_feedback_experiment_b200 import chunk_precond_kda, ops
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_oracle_with_grads

pytestmark = pytest.mark.gpu
ROWS = INPUT_NAMES[:7]
PARAMS = INPUT_NAMES[7:]
D = 128
RMS = dict(q=0.007, k=0.008, v=0.007, g=0.015, g_atk=0.015, beta_atk=0.015, beta=0.015,
           A_log=0.025, dt_bias=0.02, log_atk_scale=0.02)


def _gpu(dev, S0, A0, do, dS):
    leaves = {n: dev[n].clone().requires_grad_(True) for n in INPUT_NAMES}
    S0 = S0.clone().requires_grad_(True)
    A0 = A0.clone().requires_grad_(True)
    kw = {n: leaves[n] for n in INPUT_NAMES if n != "log_atk_scale"}
    o, S, A = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=True,
                                log_atk_scale=leaves["log_atk_scale"])
    grads = torch.autograd.grad([o, S], [leaves[n] for n in INPUT_NAMES] + [S0, A0], [do, dS])
    assert ops.last_device_status() == 0 and ops.last_backward_status() == 0
    res = dict(zip(list(INPUT_NAMES) + ["S0", "A0"], grads))
    res.update(o=o, S=S, A=A)
    return res


def _slice_against_oracle(B, T, H, b, h, seed):
    d = make_inputs(B, T, H, D, seed=seed, dist="unit", dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(seed + 1)) * 0.1
    dev = {n: d[n].cuda() for n in INPUT_NAMES}
    full = _gpu(dev, d["initial_state"].cuda(), d["initial_A_state"].cuda(), d["do"].cuda(), dS.cuda())
    assert all(torch.isfinite(t.float()).all() for t in full.values())

    sl = {n: d[n][b:b + 1, :, h:h + 1] for n in ROWS}
    sl.update(A_log=d["A_log"][h:h + 1], dt_bias=d["dt_bias"][h * D:(h + 1) * D],
              log_atk_scale=d["log_atk_scale"][h:h + 1])
    S0s, A0s = d["initial_state"][b:b + 1, h:h + 1], d["initial_A_state"][b:b + 1, h:h + 1]
    dos, dSs = d["do"][b:b + 1, :, h:h + 1], dS[b:b + 1, h:h + 1]
    ref = pkda_oracle_with_grads([sl[n] for n in INPUT_NAMES], dos, initial_state=S0s,
                                 initial_A_state=A0s, d_final_state=dSs, dtype=torch.float64)
    tag = f"B{B} T{T} ({b},{h})"
    assert rel_rms(full["o"][b:b + 1, :, h:h + 1], ref["o"]) < 0.005, tag
    assert_close(full["o"][b:b + 1, :, h:h + 1], ref["o"], 2e-2, tag + " o")
    assert_close(full["S"][b:b + 1, h:h + 1], ref["final_state"], 2e-2, tag + " S_T")
    assert_close(full["A"][b:b + 1, h:h + 1], ref["final_A_state"], 1e-4, tag + " A_T")
    for n in ROWS:
        got = full[n][b:b + 1, :, h:h + 1]
        r = rel_rms(got, ref["d" + n])
        assert r < RMS[n], f"{tag}: d{n} rel-rms {r:.3e}"
        assert_close(got, ref["d" + n], 2e-2 if n in ("q", "k", "v") else 4e-2, f"{tag} d{n}")
    assert rel_rms(full["S0"][b:b + 1, h:h + 1], ref["dinitial_state"]) < 0.01, tag
    assert rel_rms(full["A0"][b:b + 1, h:h + 1], ref["dinitial_A_state"]) < 0.02, tag

    # per-head parameter gradients: the slice alone on the GPU
    one = _gpu({n: sl[n].cuda().contiguous() for n in INPUT_NAMES}, S0s.cuda().contiguous(),
               A0s.cuda().contiguous(), dos.cuda().contiguous(), dSs.cuda().contiguous())
    for n in ("dt_bias", "log_atk_scale"):
        r = rel_rms(one[n], ref["d" + n])
        assert r < RMS[n], f"{tag}: d{n} rel-rms {r:.3e}"
    # dA_log of ONE (row, head) unit is a single number: the sum over all tokens and channels of
    # draw * softplus / sigmoid, whose terms cancel to a small remainder.  The reference's limit
    # (a relative 0.025, scripts/pkda_bench.py:46-47) is stated for a whole batch; for one unit the
    # rounding of the bf16 gate gradients shows against the cancelled sum, so the bound here adds
    # 1e-3 of the sum's absolute mass.
    z = sl["g"].double() + sl["dt_bias"].double().view(1, 1, 1, D)
    terms = ref["dg"].double() * torch.nn.functional.softplus(z) / torch.sigmoid(z)
    a, e = float(one["A_log"].double().sum()), float(ref["dA_log"].sum())
    assert abs(float(terms.sum()) - e) <= 1e-6 * float(terms.abs().sum())
    assert abs(a - e) <= RMS["A_log"] * abs(e) + 1e-3 * float(terms.abs().sum()), \
        f"{tag}: dA_log {a:.6e} vs {e:.6e} (mass {float(terms.abs().sum()):.3e})"


def test_single_gpu_configuration_slice():
    _slice_against_oracle(B=8, T=4096, H=16, b=5, h=11, seed=400)


def test_eight_gpu_configuration_per_gpu_shape_slice():
    _slice_against_oracle(B=16, T=8192, H=16, b=9, h=3, seed=410)
