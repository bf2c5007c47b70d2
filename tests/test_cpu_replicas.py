"""world_size-2 gloo test of the multi-GPU result reduction and request sharding (CPU only)."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from reef_b200 import replicas


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sums, maxes = replicas.aggregate(dist, {"inf_s": 100.0 + rank, "launches": 10 * (rank + 1)},
                                     {"ms_per_step": 1.0 + rank, "p99": 2.0 - rank})
    dist.barrier()
    if rank == 0:
        torch.save((sums, maxes), out)
    dist.destroy_process_group()


def test_aggregate_two_ranks_gloo(tmp_path):
    out = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(2, 29533, out), nprocs=2, join=True)
    sums, maxes = torch.load(out)
    assert sums == {"inf_s": 201.0, "launches": 30.0}            # whole-job totals
    assert maxes == {"ms_per_step": 2.0, "p99": 2.0}             # slowest rank


def test_single_process_passthrough_and_sharding():
    s, m = replicas.aggregate(None, {"a": 1.0}, {"b": 2.0})
    assert s == {"a": 1.0} and m == {"b": 2.0}
    parts = [replicas.shard_round_robin(10, r, 4) for r in range(4)]
    assert sorted(sum(parts, [])) == list(range(10)) and parts[1] == [1, 5, 9]
    assert replicas.device_for_rank(5, 4) == 1
