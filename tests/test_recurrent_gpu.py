"""GPU parity of the token-by-token kernel (decode step, cached prefill, exact
fp32 forward) against the reference-generated golden vectors and the oracle."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from delta_feedback_experiment_b200 import fused_recurrent_precond_kda, chunk_precond_kda
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_packed_oracle, pkda_recurrent_oracle

pytestmark = pytest.mark.gpu
CASES = ["tiny_unit", "tiny_production_state", "d64_cross_chunk_state", "d128_production",
         "d128_unit_state", "decode_steps"]


def call(fn, d, dev="cuda", **kw):
    t = {n: d[n].to(dev) for n in INPUT_NAMES}
    S0 = d.get("initial_state")
    A0 = d.get("initial_A_state")
    return fn(q=t["q"], k=t["k"], v=t["v"], g=t["g"], g_atk=t["g_atk"], beta_atk=t["beta_atk"],
              beta=t["beta"], A_log=t["A_log"], dt_bias=t["dt_bias"],
              initial_state=None if S0 is None else S0.to(dev),
              initial_A_state=None if A0 is None else A0.to(dev),
              output_final_state=True, log_atk_scale=t["log_atk_scale"], **kw)


@pytest.mark.parametrize("name", CASES)
def test_fp32_matches_reference_golden(name):
    g = load_golden(name)
    o, S, A = call(fused_recurrent_precond_kda, g)
    assert_close(o, g["o"], 1e-4, "o")
    assert_close(S, g["final_state"], 1e-4, "S")
    assert_close(A, g["final_A_state"], 1e-4, "A")


@pytest.mark.parametrize("name", ["d64_cross_chunk_state", "tiny_unit"])
def test_fp32_chunk_entry_point_uses_exact_kernel(name):
    """fp32 activations (the CPU-parity configuration) go through the exact kernel."""
    g = load_golden(name)
    o, S, A = call(chunk_precond_kda, g)
    assert_close(o, g["o"], 1e-4, "o")
    assert_close(S, g["final_state"], 1e-4, "S")


def test_config0_shape_fp32():
    """B=2, T=512, H=4, d=64, fp32, zero initial state (benchmark config 0)."""
    d = make_inputs(2, 512, 4, 64, seed=100, dist="unit", dtype=torch.float32)
    ref = pkda_recurrent_oracle(*[d[n] for n in INPUT_NAMES], dtype=torch.float64)
    o, S, A = call(chunk_precond_kda, d)
    assert_close(o, ref[0], 1e-4, "o")
    assert_close(S, ref[1], 1e-4, "S")
    assert_close(A, ref[2], 1e-4, "A")


@pytest.mark.parametrize("dist", ["unit", "production"])
def test_bf16_decode_steps_inplace(dist):
    """16 sequential single-token steps on a (B=4,H=4,d=128) slice, state updated
    in place, against the fp32 oracle fed the same bf16-rounded inputs."""
    B, T, H, D = 4, 16, 4, 128
    d = make_inputs(B, T, H, D, seed=7, dist=dist, dtype=torch.bfloat16, with_state=True)
    ref = pkda_recurrent_oracle(*[d[n] for n in INPUT_NAMES], initial_state=d["initial_state"],
                                initial_A_state=d["initial_A_state"], dtype=torch.float64)
    S = d["initial_state"].cuda().clone()
    A = d["initial_A_state"].cuda().clone()
    dev = {n: d[n].cuda() for n in INPUT_NAMES}
    outs = []
    for t in range(T):
        sl = {n: dev[n][:, t:t + 1] for n in INPUT_NAMES[:7]}
        o, S2, A2 = fused_recurrent_precond_kda(
            **sl, A_log=dev["A_log"], dt_bias=dev["dt_bias"], initial_state=S, initial_A_state=A,
            output_final_state=True, log_atk_scale=dev["log_atk_scale"], inplace_state=True)
        assert S2.data_ptr() == S.data_ptr() and A2.data_ptr() == A.data_ptr()
        outs.append(o)
    o = torch.cat(outs, 1)
    assert o.dtype == torch.bfloat16
    assert_close(o, ref[0], 2e-2, "o")          # bf16 output rounding
    assert_close(S, ref[1], 1e-4, "S")          # states stay fp32
    assert_close(A, ref[2], 1e-4, "A")


def test_packed_sequences_fp32():
    lens = [5, 1, 70, 33]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    d = make_inputs(1, offs[-1], 2, 32, seed=9, dist="production", dtype=torch.float32,
                    with_state=True, n_states=len(lens))
    ref = pkda_packed_oracle(*[d[n] for n in INPUT_NAMES], cu_seqlens=offs,
                             initial_state=d["initial_state"],
                             initial_A_state=d["initial_A_state"], dtype=torch.float64)
    o, S, A = call(fused_recurrent_precond_kda, d,
                   cu_seqlens=torch.tensor(offs, dtype=torch.int32, device="cuda"))
    assert_close(o, ref[0], 1e-4, "o")
    assert_close(S, ref[1], 1e-4, "S")
    assert_close(A, ref[2], 1e-4, "A")


def test_run_twice_is_bitwise_identical():
    d = make_inputs(2, 20, 2, 128, seed=3, dist="production", dtype=torch.bfloat16, with_state=True)
    a = call(fused_recurrent_precond_kda, d)
    b = call(fused_recurrent_precond_kda, d)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("dtype,inplace", [(torch.bfloat16, True), (torch.float32, False)])
def test_large_decode_batch(dtype, inplace):
    """Several (row, head) units per SM: two consecutive cached single-token steps, states
    carried (in place or not), against the oracle."""
    B, H, D, steps = 42, 16, 128, 2
    d = make_inputs(B, steps, H, D, seed=77, dist="production", dtype=dtype, with_state=True)
    ref_o, ref_S, ref_A = pkda_recurrent_oracle(*[d[n] for n in INPUT_NAMES],
                                                initial_state=d["initial_state"],
                                                initial_A_state=d["initial_A_state"])
    t = {n: d[n].cuda() for n in INPUT_NAMES}
    S, A = d["initial_state"].cuda(), d["initial_A_state"].cuda()
    outs = []
    for s in range(steps):
        o, S, A = fused_recurrent_precond_kda(
            **{n: t[n][:, s:s + 1].contiguous() for n in INPUT_NAMES[:7]}, A_log=t["A_log"],
            dt_bias=t["dt_bias"], initial_state=S, initial_A_state=A, output_final_state=True,
            log_atk_scale=t["log_atk_scale"], inplace_state=inplace)
        outs.append(o)
    rtol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert_close(torch.cat(outs, 1), ref_o, rtol, "o")
    assert_close(S, ref_S, 1e-4, "S")
    assert_close(A, ref_A, 1e-4, "A")
