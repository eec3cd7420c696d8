"""The no-allocation forward (``pkda_chunk_fwd_static``) against the regular
entry point.

Some hosts of this library may not allocate device memory at call time (a
serving engine with fixed pools, a plugin inside another runtime's callback).
For them the library carries a fixed scratch array; this test drives that entry
point through the C ABI with caller-owned buffers, twice in a row with different
inputs (the shared array keeps the previous call's contents), and requires the
results to be bitwise those of ``pkda_chunk_fwd``.  It also checks that a problem
beyond the array's size is refused.  Collected last on purpose."""

import pytest
import torch

from delta_feedback_experiment_b200 import ops
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

pytestmark = pytest.mark.gpu


def _buffers(q, v):
    return [torch.empty(shape, device=q.device, dtype=dt)
            for shape, dt in ops.intermediate_meta(q, v, False)]


def _run_both(seed, B, T, H):
    d = make_inputs(B, T, H, 128, seed=seed, dist="production", dtype=torch.bfloat16,
                    with_state=True)
    t = [d[n].cuda().contiguous() for n in INPUT_NAMES]
    S0, A0 = d["initial_state"].cuda(), d["initial_A_state"].cuda()
    o_ref, S_ref, A_ref, saved_ref = ops.chunk_forward(*t, 128 ** -0.5, 1.5, 1e-6, S0, A0, None, True)
    o = torch.empty_like(o_ref)
    S, A = torch.empty_like(S_ref), torch.empty_like(A_ref)
    saved = _buffers(t[0], t[2])
    ops.track_device_status(True)   # drops the 4-byte status copy the call above kept
    allocated = torch.cuda.memory_allocated()
    ops.chunk_forward_static(*t, 128 ** -0.5, 1.5, 1e-6, o, saved, S0, A0, S, A)
    assert torch.cuda.memory_allocated() == allocated  # nothing allocated through torch either
    torch.cuda.synchronize()
    assert ops.last_device_status() == 0   # read from the library's own array
    assert torch.equal(o, o_ref) and torch.equal(S, S_ref) and torch.equal(A, A_ref)
    for a, b in zip(saved, saved_ref):
        assert torch.equal(a, b)


def test_static_scratch_matches_regular_entry_point_twice():
    _run_both(seed=501, B=2, T=200, H=3)
    _run_both(seed=502, B=1, T=130, H=2)   # smaller: stale bytes of the first call remain behind it
    _run_both(seed=503, B=2, T=200, H=3)


def test_static_scratch_rejects_oversized_problem():
    B, T, H = 2, 4096, 16   # needs ~33 MiB of scratch
    d = make_inputs(1, 64, 1, 128, seed=1, dist="unit", dtype=torch.bfloat16)
    big = lambda *shape: torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    q = big(B, T, H, 128)
    sc = big(B, T, H)
    args = [q, q, q, q, torch.empty(B, T, H, device="cuda"), sc, sc,
            torch.zeros(H, device="cuda"), torch.zeros(H * 128, device="cuda"),
            torch.zeros(H, device="cuda")]
    with pytest.raises(RuntimeError, match="static scratch"):
        ops.chunk_forward_static(*args, 128 ** -0.5, 1.5, 1e-6, q, _buffers(q, q))
    assert ops.static_scratch_bytes() == 16 << 20
