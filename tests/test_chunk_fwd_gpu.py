"""GPU parity of the chunked forward (bf16, d=128) against the golden vectors,
the oracle and -- stage by stage -- the CPU model of the kernel pipeline."""

import pytest
import torch

from conftest import assert_close, load_golden, rel_rms
from delta_feedback_experiment_b200 import chunk_precond_kda, pkda_recurrence
from delta_feedback_experiment_b200 import ops
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_packed_oracle, pkda_recurrent_oracle
import chunk_model as cm

pytestmark = pytest.mark.gpu

# Relative-RMS limits the reference's own operator benchmark enforces
# (scripts/pkda_bench.py:46-47,217).
OUT_RMS = 0.005


def bf16_inputs(g):
    """Golden fp32 inputs rounded to the operator's bf16 activations."""
    d = dict(g)
    for n in ("q", "k", "v", "g", "beta", "beta_atk", "do"):
        d[n] = g[n].to(torch.bfloat16)
    return d


def run_chunk(d, cu=None, final=True):
    t = {n: d[n].cuda() for n in INPUT_NAMES}
    S0, A0 = d.get("initial_state"), d.get("initial_A_state")
    return chunk_precond_kda(
        q=t["q"], k=t["k"], v=t["v"], g=t["g"], g_atk=t["g_atk"], beta_atk=t["beta_atk"],
        beta=t["beta"], A_log=t["A_log"], dt_bias=t["dt_bias"],
        initial_state=None if S0 is None else S0.cuda(),
        initial_A_state=None if A0 is None else A0.cuda(),
        output_final_state=final, log_atk_scale=t["log_atk_scale"],
        cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32, device="cuda"))


def oracle(d, cu=None):
    ins = [d[n] for n in INPUT_NAMES]
    kw = dict(initial_state=d.get("initial_state"), initial_A_state=d.get("initial_A_state"),
              dtype=torch.float64)
    if cu is None:
        return pkda_recurrent_oracle(*ins, **kw)
    return pkda_packed_oracle(*ins, cu_seqlens=cu, **kw)


def check(o, S, A, ref, tag):
    assert o.dtype == torch.bfloat16
    assert rel_rms(o, ref[0]) < OUT_RMS, f"{tag}: o rel-rms {rel_rms(o, ref[0]):.3e}"
    assert_close(o, ref[0], 2e-2, tag + ":o")
    assert_close(S, ref[1], 2e-2, tag + ":S")
    assert_close(A, ref[2], 1e-4, tag + ":A")


@pytest.mark.parametrize("name", ["d128_production", "d128_unit_state"])
def test_golden_bf16(name):
    g = load_golden(name)
    d = bf16_inputs(g)
    ref = oracle(d)
    o, S, A = run_chunk(d)
    check(o, S, A, ref, name)
    # and against the reference's own fp32 run on unrounded inputs (looser: input rounding)
    assert rel_rms(o, g["o"]) < 2e-2


@pytest.mark.parametrize("dist", ["unit", "production"])
@pytest.mark.parametrize("T", [1, 16, 63, 64, 65, 200, 512])
def test_lengths_and_distributions(T, dist):
    d = make_inputs(2, T, 3, 128, seed=20 + T, dist=dist, dtype=torch.bfloat16, with_state=True)
    ref = oracle(d)
    o, S, A = run_chunk(d)
    check(o, S, A, ref, f"T{T}-{dist}")


def test_zero_state_no_final_state_custom_op():
    d = make_inputs(2, 256, 4, 128, seed=31, dist="unit", dtype=torch.bfloat16)
    ref = oracle(d)
    t = {n: d[n].cuda() for n in INPUT_NAMES}
    for lean in (True, False):
        o, saved = pkda_recurrence(*[t[n] for n in INPUT_NAMES], 128 ** -0.5, 1.5, 1e-6, lean)
        assert len(saved) == (6 if lean else 11)
        meta = ops.intermediate_meta(t["q"], t["v"], lean)
        for s, (shape, dt) in zip(saved, meta):
            assert tuple(s.shape) == shape and s.dtype == dt and s.is_contiguous()
        assert rel_rms(o, ref[0]) < OUT_RMS
        assert_close(o, ref[0], 2e-2, "o")


def test_packed_variable_length():
    lens = [130, 64, 1, 77, 300]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    d = make_inputs(1, offs[-1], 2, 128, seed=41, dist="production", dtype=torch.bfloat16,
                    with_state=True, n_states=len(lens))
    ref = oracle(d, offs)
    o, S, A = run_chunk(d, offs)
    check(o, S, A, ref, "packed")


def test_stage_outputs_match_cpu_model():
    """Every saved intermediate of one (row, head) against the CPU model run
    with the same bf16 rounding points."""
    B, T, H, D = 1, 192, 2, 128
    d = make_inputs(B, T, H, D, seed=51, dist="production", dtype=torch.bfloat16, with_state=True)
    t = {n: d[n].cuda() for n in INPUT_NAMES}
    o, S, A, saved = ops.chunk_forward(
        *[t[n] for n in INPUT_NAMES], 128 ** -0.5, 1.5, 1e-6,
        d["initial_state"].cuda(), d["initial_A_state"].cuda(), None, True)
    Aqk, Akk, kt, gc, a_start, sa, w, kg, v_new, h, qg = [x.float().cpu() for x in saved]
    f64 = lambda x: x.to(torch.float64)
    for hd in range(H):
        args = [f64(d[n][0, :, hd]) for n in ("q", "k", "v", "g", "g_atk", "beta_atk", "beta")]
        _, _, _, st = cm.chunk_forward(
            *args, f64(d["A_log"][hd]), f64(d["dt_bias"].view(H, D)[hd]),
            f64(d["log_atk_scale"][hd]), D ** -0.5, 1.5, 1e-6,
            f64(d["initial_state"][0, hd]), f64(d["initial_A_state"][0, hd]),
            act=torch.bfloat16, keep=True)
        for ci, ch in enumerate(st):
            lo, hi = ch["lo"], ch["hi"]
            tag = f"h{hd} c{ci} "
            assert rel_rms(kt[0, lo:hi, hd], ch["Kt"]) < 3e-3, tag + "kt"
            assert rel_rms(gc[0, ci, hd], ch["gC"]) < 1e-4, tag + "gc"
            assert rel_rms(Aqk[0, lo:hi, hd, : hi - lo], ch["P"]) < 1e-2, tag + "Aqk"
            assert rel_rms(Akk[0, lo:hi, hd, : hi - lo], ch["Tm"]) < 1e-2, tag + "Akk"
            assert rel_rms(w[0, lo:hi, hd], ch["W"]) < 1e-2, tag + "w"
            assert rel_rms(kg[0, lo:hi, hd], ch["Kg"]) < 5e-3, tag + "kg"
            assert rel_rms(qg[0, lo:hi, hd], ch["Qd"]) < 5e-3, tag + "qg"
            assert rel_rms(h[0, ci, hd], ch["h"]) < 1e-2, tag + "h"
            assert rel_rms(v_new[0, lo:hi, hd], ch["E"]) < 1e-2, tag + "v_new"


def test_device_status_word_is_clean():
    """The tcgen05 output stage bounds every wait and reports a give-up through a
    status word instead of hanging; a healthy run leaves it at zero."""
    d = make_inputs(2, 300, 2, 128, seed=62, dist="production", dtype=torch.bfloat16, with_state=True)
    o, S, A = run_chunk(d)
    assert ops.last_device_status() == 0
    check(o, S, A, oracle(d), "status")


def test_run_twice_is_bitwise_identical():
    d = make_inputs(2, 130, 2, 128, seed=61, dist="unit", dtype=torch.bfloat16, with_state=True)
    a, b = run_chunk(d), run_chunk(d)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
