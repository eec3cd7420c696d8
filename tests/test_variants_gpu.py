"""Both kernel families of a stage on the same inputs.

Single-block chunks (64 tokens, mild decay) run in the tcgen05 / tensor-memory kernels,
every other chunk in the mma.sync kernels; with unit-scale gates the second family would
see no full chunk at all.  `_lib.set_variant` pins the mma.sync kernel of a stage, so the
tests here run the same problem through each family and require (a) agreement between
the two within the bf16 parity bounds, (b) agreement of each with the float64 oracle,
and (c) on a mixed input (some chunks mild, some strongly decaying, one ragged tail) that
the default dispatch equals, bit for bit, what each family produces for its own chunks."""

import pytest
import torch

from conftest import assert_close, rel_rms
from delta_feedback_experiment_b200 import _lib, chunk_precond_kda, ops
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_oracle_with_grads

pytestmark = pytest.mark.gpu
D = 128
STAGES = ("intra_fwd", "scan_fwd", "out_fwd", "scan_bwd", "intra_bwd")
RMS = dict(q=0.007, k=0.008, v=0.007, g=0.015, g_atk=0.015, beta_atk=0.015, beta=0.015,
           A_log=0.025, dt_bias=0.02, log_atk_scale=0.02)


def _run(d, do, dS):
    leaves = {n: d[n].cuda().clone().requires_grad_(True) for n in INPUT_NAMES}
    S0 = d["initial_state"].cuda().clone().requires_grad_(True)
    A0 = d["initial_A_state"].cuda().clone().requires_grad_(True)
    kw = {n: leaves[n] for n in INPUT_NAMES if n != "log_atk_scale"}
    o, S, A = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=True,
                                log_atk_scale=leaves["log_atk_scale"])
    grads = torch.autograd.grad([o, S], [leaves[n] for n in INPUT_NAMES] + [S0, A0], [do.cuda(), dS.cuda()])
    assert ops.last_device_status() == 0 and ops.last_backward_status() == 0
    res = {"d" + n: g for n, g in zip(list(INPUT_NAMES) + ["S0", "A0"], grads)}
    res.update(o=o, S=S, A=A)
    return res


@pytest.fixture
def legacy():
    """Pins the mma.sync kernels of the listed stages for the duration of a block."""
    def pin(stages, on):
        for s in stages:
            _lib.set_variant(s, on)
    yield pin
    pin(STAGES, False)


def _problem(B, T, H, seed, dist="unit"):
    d = make_inputs(B, T, H, D, seed=seed, dist=dist, dtype=torch.bfloat16, with_state=True)
    dS = torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(seed + 1)) * 0.1
    return d, d["do"], dS


def test_intra_families_agree_with_each_other_and_the_oracle(legacy):
    # 8 x 16 (row, head) units: the scans stay on tcgen05 in both runs; only the intra kernels swap.
    B, T, H = 8, 256, 16
    d, do, dS = _problem(B, T, H, seed=41)
    new = _run(d, do, dS)
    legacy(("intra_fwd", "intra_bwd"), True)
    old = _run(d, do, dS)
    legacy(STAGES, False)
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], do, initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], d_final_state=dS, dtype=torch.float64)
    for name, got in (("tcgen05", new), ("mma.sync", old)):
        assert rel_rms(got["o"], ref["o"]) < 0.005, name
        assert_close(got["o"], ref["o"], 2e-2, f"{name} o")
        assert_close(got["S"], ref["final_state"], 2e-2, f"{name} S_T")
        assert_close(got["A"], ref["final_A_state"], 1e-4, f"{name} A_T")
        for n in INPUT_NAMES:
            r = rel_rms(got["d" + n], ref["d" + n])
            assert r < RMS[n], f"{name}: d{n} rel-rms {r:.3e}"
    # the two families against each other: same rounding points, different summation order, so
    # two bf16 roundings of nearly equal values apart (about 3e-3 relative rms for o)
    assert rel_rms(new["o"], old["o"]) < 0.005
    for n in INPUT_NAMES:
        assert rel_rms(new["d" + n], old["d" + n]) < RMS[n], n
    torch.testing.assert_close(new["A"], old["A"], rtol=1e-6, atol=1e-7)


def test_all_five_stages_pinned_to_mma_sync(legacy):
    B, T, H = 8, 192, 16
    d, do, dS = _problem(B, T, H, seed=43)
    new = _run(d, do, dS)
    legacy(STAGES, True)
    old = _run(d, do, dS)
    legacy(STAGES, False)
    assert rel_rms(new["o"], old["o"]) < 0.005
    assert rel_rms(new["S"], old["S"]) < 0.005
    for n in INPUT_NAMES:
        assert rel_rms(new["d" + n], old["d" + n]) < RMS[n], n


def test_mixed_chunks_take_their_own_kernel_bit_for_bit(legacy):
    """Rows 0..3 carry unit-scale gates (single-block chunks), rows 4..7 the strongly decaying
    gates of about 3 nats per token (hierarchy), and T = 160 leaves a ragged 32-token tail on
    every row.  The default dispatch must give rows 0..3's full chunks the tcgen05 result and everything else
    the mma.sync result; since rows are independent, the whole-batch run is compared bitwise
    with (a) itself run a second time and (b) a run whose intra stages are pinned to mma.sync."""
    B, T, H = 8, 160, 16
    d, do, dS = _problem(B, T, H, seed=45)
    # raw gate + 3: softplus gives about 3 nats per token, 280 log2 units per chunk, far past the
    # single-block limit, while rows 0..3 stay near 75 log2 units per chunk
    d["g"][4:] = (d["g"][4:].float() + 3.0).to(d["g"].dtype)
    first = _run(d, do, dS)
    again = _run(d, do, dS)
    for n in first:
        assert torch.equal(first[n], again[n]), f"{n}: two runs differ"
    # the same batch with the intra stages pinned to mma.sync: rows 4..7 ran those kernels in the
    # mixed dispatch too, so every per-row result of theirs must carry the same bits (parameter
    # gradients are sums over rows and are left out)
    legacy(("intra_fwd", "intra_bwd"), True)
    alone = _run(d, do, dS)
    legacy(STAGES, False)
    for n in ("o", "S", "A", "dq", "dk", "dv", "dg", "dbeta", "dg_atk", "dbeta_atk", "dS0", "dA0"):
        assert torch.equal(first[n][4:], alone[n][4:]), f"{n}: strongly decaying rows differ from the mma.sync run"
    # and against the oracle for the whole mixed batch
    ref = pkda_oracle_with_grads([d[n] for n in INPUT_NAMES], do, initial_state=d["initial_state"],
                                 initial_A_state=d["initial_A_state"], d_final_state=dS, dtype=torch.float64)
    assert rel_rms(first["o"], ref["o"]) < 0.005
    for n in ("q", "k", "v"):
        assert rel_rms(first["d" + n], ref["d" + n]) < RMS[n], n


def test_output_from_the_scan_equals_the_stand_alone_output_kernel(legacy):
    """By default the tcgen05 state scan also forms o (it holds the chunk-entry state and E of
    every chunk); `set_variant("out_fwd", 2)` runs the stand-alone tcgen05 output kernel on
    the h and v_new the scan stored.  Same operands, same products, same order: equal bits.
    Ragged tails (T = 200) and packed sequences included."""
    for B, T in ((8, 256), (8, 200)):
        d, do, dS = _problem(B, T, 16, seed=47)
        fused = _run(d, do, dS)
        _lib.set_variant("out_fwd", 2)
        split = _run(d, do, dS)
        _lib.set_variant("out_fwd", 0)
        for n in fused:
            assert torch.equal(fused[n], split[n]), f"T={T} {n}"
    # packed: 128 sequences x 1 head would be slow to build; 16 sequences x 8 heads = 128 units
    from delta_feedback_experiment_b200.synthetic import packed_lengths
    H = 8
    offs = packed_lengths(16 * 150, 100, 200, seed=3)[:17]
    total = offs[-1]
    d = make_inputs(1, total, H, D, seed=49, dtype=torch.bfloat16, with_state=True, n_states=len(offs) - 1)
    cu = torch.tensor(offs, dtype=torch.int32, device="cuda")

    def run():
        kw = {n: d[n].cuda() for n in INPUT_NAMES if n != "log_atk_scale"}
        o, S, A = chunk_precond_kda(**kw, initial_state=d["initial_state"].cuda(),
                                    initial_A_state=d["initial_A_state"].cuda(), output_final_state=True,
                                    log_atk_scale=d["log_atk_scale"].cuda(), cu_seqlens=cu)
        assert ops.last_device_status() == 0
        return o, S
    o1, S1 = run()
    _lib.set_variant("out_fwd", 2)
    o2, S2 = run()
    _lib.set_variant("out_fwd", 0)
    assert torch.equal(o1, o2) and torch.equal(S1, S2)
