"""GPU test of the recurrence dispatcher ``pkda_cuda_recurrence``, the free-function form of
``PreconditionedKDA._cuda_recurrence`` (reference ``delta_feedback_experiment/pkda.py:412-475``):
each of its three branches runs, is the branch the reference would take, and matches the
CPU oracle."""

import pytest
import torch

from conftest import assert_close, rel_rms
from delta_feedback_experiment_b200 import _lib, pkda_cuda_recurrence
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_recurrent_oracle

pytestmark = pytest.mark.gpu
D = 128


def _call(d, state, a_state, output_final_state, training):
    c = {n: d[n].cuda() for n in INPUT_NAMES}
    _lib.stage_timing(True)
    try:
        out = pkda_cuda_recurrence(
            c["q"], c["k"], c["v"], c["g"], c["beta"], c["g_atk"], c["beta_atk"],
            None if state is None else state.cuda(), None if a_state is None else a_state.cuda(),
            output_final_state, A_log=c["A_log"], dt_bias=c["dt_bias"],
            log_precond_center=c["log_atk_scale"], head_dim=D, training=training)
        torch.cuda.synchronize()
        stages = set(_lib.stage_timing_read())
    finally:
        _lib.stage_timing(False)
    return out, stages


def _oracle(d, state, a_state):
    return pkda_recurrent_oracle(*[d[n] for n in INPUT_NAMES], initial_state=state,
                                 initial_A_state=a_state, dtype=torch.float64)


def test_no_state_takes_the_custom_operator():
    """state None, a_state None, no final state: the dense training / prefill operator."""
    d = make_inputs(2, 130, 2, D, seed=301, dist="production", dtype=torch.bfloat16)
    (o, S, A), stages = _call(d, None, None, False, training=True)
    assert S is None and A is None
    assert "intra_fwd" in stages and "recurrent" not in stages and "decode_step" not in stages
    ref_o, _, _ = _oracle(d, None, None)
    assert rel_rms(o, ref_o) < 0.005
    assert_close(o, ref_o, 2e-2, "o")


@pytest.mark.parametrize("T", [1, 64])
def test_short_cached_prefill_takes_the_recurrent_kernel(T):
    """output_final_state, T <= 64, not training: the token-by-token kernel."""
    d = make_inputs(2, T, 2, D, seed=302 + T, dist="unit", dtype=torch.bfloat16, with_state=True)
    (o, S, A), stages = _call(d, d["initial_state"], d["initial_A_state"], True, training=False)
    assert "intra_fwd" not in stages and stages & {"recurrent", "decode_step"}
    ref_o, ref_S, ref_A = _oracle(d, d["initial_state"], d["initial_A_state"])
    assert_close(o, ref_o, 2e-2, "o")
    assert_close(S, ref_S, 1e-4, "S")
    assert_close(A, ref_A, 1e-4, "A")


@pytest.mark.parametrize("case", ["long", "training", "state_without_final"])
def test_everything_else_takes_the_chunked_kernels(case):
    """State given, but T > 64, or training, or no final state wanted: chunk_precond_kda."""
    T = 200 if case == "long" else 48
    d = make_inputs(2, T, 2, D, seed=310, dist="unit", dtype=torch.bfloat16, with_state=True)
    final = case != "state_without_final"
    (o, S, A), stages = _call(d, d["initial_state"], d["initial_A_state"], final,
                              training=case == "training")
    assert "intra_fwd" in stages and "recurrent" not in stages
    ref_o, ref_S, ref_A = _oracle(d, d["initial_state"], d["initial_A_state"])
    assert_close(o, ref_o, 2e-2, "o")
    if final:
        assert_close(S, ref_S, 2e-2, "S")
        assert_close(A, ref_A, 1e-4, "A")
    else:
        assert S is None and A is None


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensors_on_a_device_that_is_not_current():
    """The launchers make the tensors' device current themselves (the reference's kernels guard
    the same way); arguments spread over two devices are rejected before any launch."""
    d = make_inputs(1, 70, 2, D, seed=320, dist="unit", dtype=torch.bfloat16)
    ref_o, _, _ = _oracle(d, None, None)
    c = {n: d[n].to("cuda:1") for n in INPUT_NAMES}
    assert torch.cuda.current_device() == 0
    o, _, _ = pkda_cuda_recurrence(
        c["q"], c["k"], c["v"], c["g"], c["beta"], c["g_atk"], c["beta_atk"], None, None, False,
        A_log=c["A_log"], dt_bias=c["dt_bias"], log_precond_center=c["log_atk_scale"], head_dim=D)
    assert o.device == c["q"].device
    assert_close(o, ref_o, 2e-2, "o")
    with pytest.raises(RuntimeError, match="different devices"):
        pkda_cuda_recurrence(
            c["q"], c["k"].to("cuda:0"), c["v"], c["g"], c["beta"], c["g_atk"], c["beta_atk"], None, None,
            False, A_log=c["A_log"], dt_bias=c["dt_bias"], log_precond_center=c["log_atk_scale"],
            head_dim=D)
