"""The sharding helpers through the CUDA operator on one GPU: the shards of a plan are run
one after the other, merged, and compared with the unsharded call.  Row tensors must be
equal bit for bit (rows and heads are independent, and no kernel is chosen from the size of
the problem); the per-head parameter gradients are sums over rows and are compared within
rounding."""

import pytest
import torch

from conftest import rel_rms
from delta_feedback_experiment_b200 import chunk_precond_kda, ops, sharding
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs

pytestmark = pytest.mark.gpu
D = 128


def _run(inp, cu=None):
    leaves = {n: inp[n].cuda().clone().requires_grad_(True) for n in INPUT_NAMES}
    S0 = inp["initial_state"].cuda().clone().requires_grad_(True)
    A0 = inp["initial_A_state"].cuda().clone().requires_grad_(True)
    kw = {n: leaves[n] for n in INPUT_NAMES if n != "log_atk_scale"}
    o, S, A = chunk_precond_kda(**kw, initial_state=S0, initial_A_state=A0, output_final_state=True,
                                log_atk_scale=leaves["log_atk_scale"], cu_seqlens=cu)
    grads = torch.autograd.grad(o, [leaves[n] for n in INPUT_NAMES] + [S0, A0], inp["do"].cuda())
    assert ops.last_device_status() == 0 and ops.last_backward_status() == 0
    res = {"d" + n: g for n, g in zip(list(INPUT_NAMES) + ["S0", "A0"], grads)}
    res.update(o=o, S=S, A=A)
    return res


def _merge(parts, plan, H, packed=False):
    out = {}
    for n in ("o", "dq", "dk", "dv", "dg", "dg_atk", "dbeta_atk", "dbeta"):
        out[n] = sharding.merge_row_outputs([p[n] for p in parts], plan, packed=packed)
    for n in ("S", "A", "dS0", "dA0"):
        out[n] = sharding.merge_state_outputs([p[n] for p in parts], plan)
    out["dA_log"] = sharding.merge_head_grads([p["dA_log"] for p in parts], plan, H)
    out["dlog_atk_scale"] = sharding.merge_head_grads([p["dlog_atk_scale"] for p in parts], plan, H)
    out["ddt_bias"] = sharding.merge_head_grads([p["ddt_bias"] for p in parts], plan, H, per_head=D)
    return out


@pytest.mark.parametrize("B,H,world", [(16, 16, 2), (8, 32, 2), (8, 32, 16), (4, 8, 4)])
def test_sharded_equals_unsharded(B, H, world):
    # (8, 32, 16): fewer rows than ranks, so pairs of ranks split a row's heads; (4, 8, 4): shards of
    # 8 (row, head) units.  No kernel is chosen from the size of the problem, so shards of any
    # size reproduce the whole problem's bits.
    T = 192
    d = make_inputs(B, T, H, D, seed=61, dtype=torch.bfloat16, with_state=True)
    whole = _run(d)
    plan = sharding.shard_plan(B, H, world)
    parts = [_run(sharding.shard_inputs(d, sh, D)[0]) for sh in plan]
    got = _merge(parts, plan, H)
    for n in ("o", "S", "A", "dq", "dk", "dv", "dg", "dg_atk", "dbeta_atk", "dbeta", "dS0", "dA0"):
        assert got[n].shape == whole[n].shape, n
        assert torch.equal(got[n], whole[n]), f"{n}: a shard's rows differ from the whole problem's"
    for n, lim in (("dA_log", 0.025), ("ddt_bias", 0.02), ("dlog_atk_scale", 0.02)):
        assert rel_rms(got[n], whole[n].float()) < lim, n


def test_packed_batch_sharded_at_sequence_boundaries():
    H = 16
    offs = [0]
    for n in (300, 64, 129, 500, 77, 210, 333, 96, 180, 250, 400, 61, 145, 90, 270, 310):
        offs.append(offs[-1] + n)
    total, N = offs[-1], len(offs) - 1
    d = make_inputs(1, total, H, D, seed=63, dtype=torch.bfloat16, with_state=True, n_states=N)
    cu = torch.tensor(offs, dtype=torch.int32, device="cuda")
    whole = _run(d, cu)
    lengths = [offs[i + 1] - offs[i] for i in range(N)]
    plan = sharding.shard_plan(N, H, 2, seq_lengths=lengths)
    tokens = [sum(lengths[s.row0:s.row1]) for s in plan]
    assert abs(tokens[0] - tokens[1]) <= max(lengths)   # balanced by tokens, not by sequence count
    parts = []
    for sh in plan:
        mine, my_cu = sharding.shard_inputs(d, sh, D, cu_seqlens=cu.cpu())
        parts.append(_run(mine, my_cu.cuda()))
    got = _merge(parts, plan, H, packed=True)
    for n in ("o", "dq", "dk", "dv", "dg", "dg_atk", "dbeta_atk", "dbeta", "S", "A", "dS0", "dA0"):
        assert got[n].shape == whole[n].shape, n
        assert torch.equal(got[n], whole[n]), n
