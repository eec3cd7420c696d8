"""World-size-2 gloo check of the host-side multi-rank bookkeeping the benchmark
relies on: per-rank seeds give different shards, the aggregate is the sum of the
per-rank units over the MAX of the per-rank times, and sharding a batch by rows
reproduces the unsharded oracle result (the path needs no collective)."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

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
