"""World-size-2 gloo checks of the host-side multi-rank logic: the package's own
sharding helpers (`sharding.shard_plan`, `shard_inputs`, the merge functions) cut a
problem by rows, by heads and -- for a packed batch -- at sequence boundaries, each
rank runs the operator's CPU oracle on its slice, and the gathered result equals the
unsharded one (the path needs no collective); plus the benchmark's bookkeeping: per-rank
seeds give different shards, the aggregate is the sum of the per-rank units over the
MAX of the per-rank times."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from delta_feedback_experiment_b200 import sharding
from delta_feedback_experiment_b200.synthetic import INPUT_NAMES, make_inputs
from oracle.pkda_oracle import pkda_recurrent_oracle


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, T, H, D = 4, 12, 2, 16
    full = make_inputs(B, T, H, D, seed=5, dist="unit", dtype=torch.float32)
    rows = slice(rank * B // world, (rank + 1) * B // world)
    shard = [full[n][rows] if full[n].dim() >= 3 else full[n] for n in INPUT_NAMES]
    o, S, A = pkda_recurrent_oracle(*shard)
    gathered = [torch.empty_like(o) for _ in range(world)]
    dist.all_gather(gathered, o)
    # timing rule: max over ranks; units: sum over ranks
    t = torch.tensor([1.0 + rank])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    units = torch.tensor([float(o.shape[0] * T)])
    dist.all_reduce(units)
    if rank == 0:
        torch.save({"o": torch.cat(gathered, 0), "tmax": t, "units": units},
                   os.path.join(out_dir, "out.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_rows_without_collective(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = torch.load(os.path.join(tmp_path, "out.pt"))
    full = make_inputs(4, 12, 2, 16, seed=5, dist="unit", dtype=torch.float32)
    o, _, _ = pkda_recurrent_oracle(*[full[n] for n in INPUT_NAMES])
    assert torch.allclose(res["o"], o, atol=1e-6)
    assert float(res["tmax"]) == 2.0 and float(res["units"]) == 48.0


def test_per_rank_seeds_differ():
    a = make_inputs(1, 8, 1, 16, seed=1000, dist="unit")
    b = make_inputs(1, 8, 1, 16, seed=1001, dist="unit")
    assert not torch.equal(a["q"], b["q"])


def _shard_worker(rank: int, world: int, port: int, out_dir: str, B: int, H: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    T, D = 10, 16
    full = make_inputs(B, T, H, D, seed=9, dist="unit", dtype=torch.float32, with_state=True)
    plan = sharding.shard_plan(B, H, world)
    mine, _ = sharding.shard_inputs(full, plan[rank], D)
    o, S, A = pkda_recurrent_oracle(*[mine[n] for n in INPUT_NAMES], initial_state=mine["initial_state"],
                                    initial_A_state=mine["initial_A_state"])
    outs = [None] * world
    dist.all_gather_object(outs, (o, S, A))   # shards may differ in shape: gather as objects
    if rank == 0:
        torch.save({"o": sharding.merge_row_outputs([x[0] for x in outs], plan),
                    "S": sharding.merge_state_outputs([x[1] for x in outs], plan),
                    "A": sharding.merge_state_outputs([x[2] for x in outs], plan)},
                   os.path.join(out_dir, f"shard_{B}_{H}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _check_sharded(tmp_path, B, H):
    world = 2
    mp.spawn(_shard_worker, args=(world, _free_port(), str(tmp_path), B, H), nprocs=world, join=True)
    res = torch.load(os.path.join(tmp_path, f"shard_{B}_{H}.pt"))
    full = make_inputs(B, 10, H, 16, seed=9, dist="unit", dtype=torch.float32, with_state=True)
    o, S, A = pkda_recurrent_oracle(*[full[n] for n in INPUT_NAMES], initial_state=full["initial_state"],
                                    initial_A_state=full["initial_A_state"])
    assert torch.allclose(res["o"], o, atol=1e-6) and res["o"].shape == o.shape
    assert torch.allclose(res["S"], S, atol=1e-6) and torch.allclose(res["A"], A, atol=1e-6)


def test_two_ranks_shard_by_rows_with_the_package_helpers(tmp_path):
    _check_sharded(tmp_path, B=3, H=2)   # uneven rows: 1 + 2


def test_two_ranks_shard_one_row_by_heads(tmp_path):
    _check_sharded(tmp_path, B=1, H=4)   # fewer rows than ranks: the heads are split


def test_shard_plan_arithmetic():
    plan = sharding.shard_plan(8, 16, 4)
    assert [(s.row0, s.row1, s.head0, s.head1) for s in plan] == [(0, 2, 0, 16), (2, 4, 0, 16), (4, 6, 0, 16), (6, 8, 0, 16)]
    plan = sharding.shard_plan(2, 16, 8)
    assert [(s.row0, s.head0, s.head1) for s in plan] == [(0, 0, 4), (0, 4, 8), (0, 8, 12), (0, 12, 16),
                                                          (1, 0, 4), (1, 4, 8), (1, 8, 12), (1, 12, 16)]
    # packed: sequences of 100, 10, 10, 10, 100, 10 tokens over 2 ranks -> 120 + 120
    plan = sharding.shard_plan(6, 4, 2, seq_lengths=[100, 10, 10, 10, 100, 10])
    assert [(s.row0, s.row1) for s in plan] == [(0, 3), (3, 6)]
    # one long sequence: the other ranks get what is left, possibly nothing, and every sequence is owned once
    plan = sharding.shard_plan(3, 4, 3, seq_lengths=[1000, 5, 5])
    owned = [i for s in plan for i in range(s.row0, s.row1)]
    assert owned == [0, 1, 2]
    import pytest
    with pytest.raises(ValueError):
        sharding.shard_plan(3, 16, 8)     # 8 ranks cannot split 3 rows by heads
    with pytest.raises(ValueError):
        sharding.shard_plan(2, 6, 8)      # 6 heads do not divide over 4 ranks per row


def test_packed_shards_follow_sequence_boundaries():
    H, D = 2, 16
    lengths = [7, 12, 5, 9]
    offs = [0]
    for n in lengths:
        offs.append(offs[-1] + n)
    total = offs[-1]
    full = make_inputs(1, total, H, D, seed=11, dist="unit", dtype=torch.float32, with_state=True, n_states=4)
    cu = torch.tensor(offs, dtype=torch.int32)
    plan = sharding.shard_plan(4, H, 2, seq_lengths=lengths)
    pieces, states = [], []
    for sh in plan:
        mine, my_cu = sharding.shard_inputs(full, sh, D, cu_seqlens=cu)
        assert my_cu[0] == 0 and int(my_cu[-1]) == mine["q"].shape[1]
        outs, fin = [], []
        for i in range(len(my_cu) - 1):   # the oracle takes one sequence at a time
            a, b = int(my_cu[i]), int(my_cu[i + 1])
            seq = [mine[n][:, a:b] if mine[n].dim() >= 3 else mine[n] for n in INPUT_NAMES]
            o, S, _ = pkda_recurrent_oracle(*seq, initial_state=mine["initial_state"][i:i + 1],
                                            initial_A_state=mine["initial_A_state"][i:i + 1])
            outs.append(o)
            fin.append(S)
        pieces.append(torch.cat(outs, 1))
        states.append(torch.cat(fin, 0))
    got = sharding.merge_row_outputs(pieces, plan, packed=True)
    gotS = sharding.merge_state_outputs(states, plan)
    ref, refS = [], []
    for i in range(4):
        a, b = offs[i], offs[i + 1]
        seq = [full[n][:, a:b] if full[n].dim() >= 3 else full[n] for n in INPUT_NAMES]
        o, S, _ = pkda_recurrent_oracle(*seq, initial_state=full["initial_state"][i:i + 1],
                                        initial_A_state=full["initial_A_state"][i:i + 1])
        ref.append(o)
        refS.append(S)
    assert torch.equal(got, torch.cat(ref, 1)) and torch.equal(gotS, torch.cat(refS, 0))
