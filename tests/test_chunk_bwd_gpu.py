"""GPU parity of the chunked backward (bf16, d=128): all ten input gradients and
the two initial-state gradients against the autograd oracle."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from delta_feedback_experiment_b200 import _lib, chunk_precond_kda, pkda_recurrence
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_oracle_with_grads

pytestmark = pytest.mark.gpu

# Relative-RMS limits of the reference's operator benchmark (scripts/pkda_bench.py:46-47).
RMS_LIMITS = dict(zip(INPUT_NAMES, (0.007, 0.008, 0.007, 0.015, 0.015, 0.015, 0.015, 0.025, 0.02, 0.02)))
FP32_GRADS = ("g_atk", "A_log", "dt_bias", "log_atk_scale")


def run(d, cu=None, with_state=True, dS=None, lean=True):
    leaves = {n: d[n].cuda().requires_grad_(True) for n in INPUT_NAMES}
    S0 = A0 = None
    if with_state:
        S0 = d["initial_state"].cuda().requires_grad_(True)
        A0 = d["initial_A_state"].cuda().requires_grad_(True)
    o, S, A = chunk_precond_kda(
        q=leaves["q"], k=leaves["k"], v=leaves["v"], g=leaves["g"], g_atk=leaves["g_atk"],
        beta_atk=leaves["beta_atk"], beta=leaves["beta"], A_log=leaves["A_log"],
        dt_bias=leaves["dt_bias"], initial_state=S0, initial_A_state=A0,
        output_final_state=dS is not None, log_atk_scale=leaves["log_atk_scale"],
        disable_recompute=not lean,
        cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda"))
    loss = (o.float() * d["do"].cuda().float()).sum()
    if dS is not None:
        loss = loss + (S * dS.cuda()).sum()
    wrt = list(leaves.values()) + ([S0, A0] if with_state else [])
    grads = torch.autograd.grad(loss, wrt)
    out = {"d" + n: g for n, g in zip(INPUT_NAMES, grads)}
    if with_state:
        out["dinitial_state"], out["dinitial_A_state"] = grads[10], grads[11]
    out["o"] = o
    return out


def check(res, ref, tag):
    from delta_feedback_experiment_b200 import ops
    assert ops.last_backward_status() == 0, f"{tag}: a bounded wait in a backward kernel gave up"
    for n in INPUT_NAMES:
        a, e = res["d" + n], ref["d" + n]
        assert a.dtype == (torch.float32 if n in FP32_GRADS else torch.bfloat16), n
        r = rel_rms(a, e)
        assert r < RMS_LIMITS[n], f"{tag}: d{n} rel-rms {r:.3e} >= {RMS_LIMITS[n]}"
        if n not in ("A_log", "dt_bias", "log_atk_scale"):
            assert_close(a, e, 2e-2 if n in ("q", "k", "v") else 4e-2, f"{tag}:d{n}")
    for n in ("dinitial_state", "dinitial_A_state"):
        if n in ref and n in res:
            assert rel_rms(res[n], ref[n]) < 0.01, f"{tag}: {n} {rel_rms(res[n], ref[n]):.3e}"


@pytest.mark.parametrize("dist", ["unit", "production"])
@pytest.mark.parametrize("T", [64, 200, 256])
def test_gradients_with_state(T, dist):
    B, H, D = 2, 2, 128
    d = make_inputs(B, T, H, D, seed=70 + T, dist=dist, dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(5)) * 0.1
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], d_final_state=dS,
                                 dtype=torch.float64)
    res = run(d, dS=dS)
    check(res, ref, f"T{T}-{dist}")


@pytest.mark.parametrize("T", [1, 17, 65])
def test_short_and_partial_chunks(T):
    d = make_inputs(2, T, 2, 128, seed=90 + T, dist="unit", dtype=torch.bfloat16, with_state=True)
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], dtype=torch.float64)
    res = run(d)
    for n in ("q", "k", "v", "beta"):
        assert rel_rms(res["d" + n], ref["d" + n]) < 0.015, n
    assert rel_rms(res["dinitial_state"], ref["dinitial_state"]) < 0.01


@pytest.mark.parametrize("name", ["d128_production", "d128_unit_state"])
def test_golden_inputs(name):
    g = load_golden(name)
    d = dict(g)
    for n in ("q", "k", "v", "g", "beta", "beta_atk", "do"):
        d[n] = g[n].to(torch.bfloat16)
    ws = "initial_state" in g
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d.get("initial_state"),
                                 initial_A_state=d.get("initial_A_state"),
                                 d_final_state=g["d_final_state"], dtype=torch.float64)
    res = run(d, with_state=ws, dS=g["d_final_state"])
    check(res, ref, name)
    # against the reference's own fp32 gradients on unrounded inputs (adds input rounding)
    for n in ("q", "k", "v"):
        assert rel_rms(res["d" + n], g["d" + n]) < 3e-2, n


def test_custom_op_all_ten_gradients_lean_equals_full():
    """The training entry point (no state): autograd.grad of all ten inputs, FP32
    for the learned vectors and the preconditioner gate
    (scripts/pkda_bench.py:190-202), lean and retaining backward bitwise equal."""
    d = make_inputs(2, 320, 3, 128, seed=77, dist="production", dtype=torch.bfloat16)
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"], dtype=torch.float64)
    results = []
    for lean in (False, True):
        leaves = [d[n].cuda().requires_grad_(True) for n in INPUT_NAMES]
        o, _saved = pkda_recurrence(*leaves, 128 ** -0.5, 1.5, 1e-6, lean)
        grads = torch.autograd.grad(o, leaves, d["do"].cuda())
        results.append(grads)
        res = {"d" + n: g for n, g in zip(INPUT_NAMES, grads)}
        check(res, ref, f"lean={lean}")
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_packed_variable_length_gradients():
    lens = [130, 64, 1, 77, 200]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    d = make_inputs(1, offs[-1], 2, 128, seed=81, dist="unit", dtype=torch.bfloat16,
                    with_state=True, n_states=len(lens))
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], cu_seqlens=offs,
                                 dtype=torch.float64)
    res = run(d, cu=offs)
    check(res, ref, "packed")


def test_packed_ragged_sequences_on_the_tensor_memory_scans():
    """Eight ragged sequences x sixteen heads = 128 (sequence, head) units: enough for the
    forward and backward state scans to take their tcgen05 / tensor-memory kernels (one CTA
    per unit, all 128 value columns).  Ragged last chunks, a one-token sequence and a
    cotangent on the final state, against the float64 oracle."""
    lens = [130, 64, 1, 77, 200, 65, 127, 190]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    H, D = 16, 128
    d = make_inputs(1, offs[-1], H, D, seed=85, dist="unit", dtype=torch.bfloat16,
                    with_state=True, n_states=len(lens))
    dS = torch.randn(len(lens), H, D, D, generator=torch.Generator().manual_seed(9)) * 0.1
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], cu_seqlens=offs,
                                 d_final_state=dS, dtype=torch.float64)
    res = run(d, cu=offs, dS=dS)
    assert rel_rms(res["o"], ref["o"]) < 0.005
    check(res, ref, "packed-128-units")


def test_backward_twice_is_bitwise_identical():
    d = make_inputs(2, 150, 2, 128, seed=83, dist="production", dtype=torch.bfloat16, with_state=True)
    a, b = run(d), run(d)
    for key in a:
        assert torch.equal(a[key], b[key]), key


@pytest.mark.parametrize("cap", [1, 2, 4, 8, 16, 32, 64])
@pytest.mark.parametrize("dist", ["unit", "production"])
def test_direct_block_variants(cap, dist):
    """The kernels pair tokens through one reference row per block of b tokens when
    the decay allows it and through the reference-row hierarchy otherwise; every
    cap on b must give the same forward and gradients within tolerance."""
    from delta_feedback_experiment_b200 import _lib
    d = make_inputs(2, 192, 2, 128, seed=95, dist=dist, dtype=torch.bfloat16, with_state=True)
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], d["do"],
                                 initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], dtype=torch.float64)
    _lib.set_direct_block_cap(cap)
    try:
        res = run(d)
    finally:
        _lib.set_direct_block_cap(64)
    assert rel_rms(res["o"], ref["o"]) < 0.005
    check(res, ref, f"cap{cap}-{dist}")


@pytest.mark.parametrize("B", [4, 8])
def test_wide_state_slices_match_narrow_ones(B):
    """The state scans have two implementations: tcgen05 / tensor-memory kernels (one CTA per
    (row, head), all 128 value columns; the default at every size) and mma.sync kernels that
    cut the value columns into 32- or 64-wide slices when there are fewer than 120 (row, head)
    units (`set_variant("scan_fwd" / "scan_bwd", 1)`).  Rows are independent, so a row of the
    big batch must agree with the same row run alone through the other implementation.
    Both feed the same bf16 operands to the tensor cores in the same order; on this short input
    every result is equal bit for bit, which this test pins.  That is a property of the input,
    not a guarantee: the tcgen05 scan adds U inside the fp32 accumulator while the mma.sync
    scan subtracts in a register, and on long inputs a few outputs differ by one bf16 unit in
    the last place (T = 1024: max |delta o| = 3.8e-6 with every gradient and the final state
    still equal), which is why the full-size tests compare within tolerance.  A row run alone
    through the default kernels must equal the batch in any case."""
    H, T = 16, 130
    d = make_inputs(B, T, H, 128, seed=97, dist="production", dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, 128, 128, generator=torch.Generator().manual_seed(6)) * 0.1
    full = run(d, dS=dS)
    for b in range(0, B, 3):
        one = {k: (v[b:b + 1] if torch.is_tensor(v) and v.dim() >= 3 and v.shape[0] == B else v)
               for k, v in d.items()}
        same = run(one, dS=dS[b:b + 1])
        _lib.set_variant("scan_fwd", 1)
        _lib.set_variant("scan_bwd", 1)
        try:
            part = run(one, dS=dS[b:b + 1])
        finally:
            _lib.set_variant("scan_fwd", 0)
            _lib.set_variant("scan_bwd", 0)
        for key in ("o", "dq", "dk", "dv", "dg", "dbeta", "dg_atk", "dbeta_atk", "dinitial_state"):
            assert torch.equal(full[key][b:b + 1], same[key]), (b, key, "default kernels")
            assert torch.equal(full[key][b:b + 1], part[key]), (b, key, "sliced mma.sync scans")
