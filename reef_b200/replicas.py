"""Multi-GPU layout of the executor path: independent replicas, no data-path collective.

The reference is single-GPU (src/reef/executor/executor_base.cpp:19-22 always picks device 0).  Requests are
independent units, so N GPUs run N schedulers, each with a full weight replica and its own clients; a front
end shards requests round-robin (real-time) or by client affinity (best-effort).  The only cross-rank
traffic is the benchmark's own barrier and the reduction of its results, implemented here so that it can be
tested on CPU with the gloo backend.
"""
from __future__ import annotations


def device_for_rank(local_rank: int, device_count: int) -> int:
    """One process per GPU: rank r drives device r (mod the visible devices)."""
    if device_count <= 0:
        raise ValueError("no device")
    return local_rank % device_count


def shard_round_robin(num_requests: int, rank: int, world: int) -> list:
    """Indices of the requests rank `rank` serves when a front end deals them round-robin."""
    return list(range(rank, num_requests, world))


def aggregate(dist, sums: dict, maxes: dict, device=None) -> tuple:
    """All-reduce of per-rank results: `sums` (throughputs, launch counts) are added over ranks, `maxes`
    (times, latencies) take the slowest rank.  `dist` is torch.distributed or None (single process)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return dict(sums), dict(maxes)
    import torch
    ks, km = sorted(sums), sorted(maxes)
    ts = torch.tensor([float(sums[k]) for k in ks], dtype=torch.float64, device=device)
    tm = torch.tensor([float(maxes[k]) for k in km], dtype=torch.float64, device=device)
    if ts.numel():
        dist.all_reduce(ts, op=dist.ReduceOp.SUM)
    if tm.numel():
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    return {k: float(v) for k, v in zip(ks, ts.tolist())}, {k: float(v) for k, v in zip(km, tm.tolist())}
