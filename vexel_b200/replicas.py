"""Request sharding over independent replicas: one process per GPU, no collective on the data path.

The reference schedules every sequence on one device (inference/scheduler/scheduler.go:245, the Run loop
owns one runtime and one cache).  Sequences never exchange data, so N GPUs run N copies of that loop,
each with its own weights, block pool and scheduler, and a request is owned by exactly one of them from
admission to completion.  The only cross-rank traffic is control: a barrier around a timed region and a
max-reduction of the per-rank durations.  `torch.distributed` carries both (NCCL on GPUs, gloo on CPU).
"""
import os

import numpy as np


def rank_env():
    """(world, rank, local_rank) from the launcher's environment; (1, 0, 0) when launched plainly."""
    return (int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")))


def init(backend="nccl", local_rank=0):
    """Joins the process group when the launcher started more than one rank.  Returns torch.distributed or None."""
    world, _, _ = rank_env()
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group(backend)
    return dist


def owner_of(request_id, world):
    """The replica that owns a request for its whole life (its KV blocks live in that replica's pool only)."""
    return int(request_id) % int(world)


def shard(request_ids, world, rank):
    """The requests this replica admits, in arrival order.  Shards are disjoint and cover every request."""
    ids = np.asarray(request_ids, dtype=np.int64)
    return ids[(ids % world) == rank]


def rank_seeds(rank, base=0):
    """Distinct synthetic-data seeds per replica: (workload rng, weights, free-list shuffle, KV fill stride)."""
    return {"workload": base + 2 + rank, "weights": base + rank, "free_list": base + 3 + rank, "kv_fill": 1000 * rank}


def _device_for(dist, local_rank):
    import torch
    return torch.device("cuda", local_rank) if dist.get_backend() == "nccl" else torch.device("cpu")


def barrier(dist):
    if dist is not None:
        dist.barrier()


def max_over_ranks(dist, value, local_rank=0):
    """The slowest replica's value: a whole-job duration is the maximum over ranks, never the mean."""
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=_device_for(dist, local_rank))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, value, local_rank=0):
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=_device_for(dist, local_rank))
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def job_throughput(dist, units_this_rank, seconds_this_rank, local_rank=0):
    """Units all replicas processed divided by the slowest replica's time."""
    total = sum_over_ranks(dist, units_this_rank, local_rank)
    slowest = max_over_ranks(dist, seconds_this_rank, local_rank)
    return total / slowest, slowest


def shutdown(dist):
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
