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


class Dispatcher:
    """Places every arriving request on the replica with the most free KV blocks, for the request's whole life.

    The reference admits every request into its one cache (Scheduler.AddSequence, inference/scheduler/scheduler.go:645-676).
    With one cache per GPU the admission step gains a choice; a request's cost to a replica is the blocks its context will
    hold, and a decode step lasts as long as the replica with the most resident KV, so the router keeps the free-block counts
    level: most free blocks first, fewest resident sequences on a tie, lowest rank after that (`place` says what changes when
    a replica's batch size is capped).  The decision is a pure
    function of the arrival stream, so every rank that replays the same stream reaches the same placement without
    talking to the others; `refresh` replaces the book-keeping by the replicas' measured free-block counts (one
    all-gather) where lengths are not known in advance.
    """

    def __init__(self, world, blocks_per_replica, max_seqs_per_replica=0, block_tokens=16):
        self.world, self.block_tokens = int(world), int(block_tokens)
        self.free = [int(blocks_per_replica)] * self.world
        self.used = [0] * self.world          # blocks held by the requests placed on each replica
        self.seqs = [0] * self.world
        self.max_seqs = int(max_seqs_per_replica)
        self.placed = {}                      # request id -> (rank, blocks)

    def blocks_for(self, tokens):
        return (int(tokens) + self.block_tokens - 1) // self.block_tokens

    def place(self, request_id, tokens):
        """Returns the owning rank, or -1 when no replica can hold the request now (the caller queues it).

        Without a per-replica sequence limit: the replica with the most free blocks.  With one (a replica's batch is capped,
        e.g. at the 64 rows the projections' fast path covers), a replica that fills its slots with short requests could not
        take its share of the long ones later, so the choice is made among the replicas with the fewest sequences (at most one
        more than the emptiest) so that the total squared deviation of the replicas' loads from the running mean
        load per sequence grows least."""
        need = self.blocks_for(tokens)
        cand = [r for r in range(self.world) if self.free[r] >= need and not (self.max_seqs and self.seqs[r] >= self.max_seqs)]
        if not cand:
            return -1
        if self.max_seqs:
            fewest = min(self.seqs[r] for r in cand)
            cand = [r for r in cand if self.seqs[r] <= fewest + 1]
            n_placed = sum(self.seqs) + 1
            mean = (sum(self.used) + need) / n_placed
            # deviation of a replica from the mean load for its sequence count: d_r = used_r - mean * seqs_r.  Adding a request
            # that is (need - mean) above the mean changes sum(d_r^2) by 2 d_r (need - mean) + const: a request heavier than
            # the mean goes to the most under-loaded candidate, a lighter one to the most over-loaded
            best = min(cand, key=lambda r: ((self.used[r] - mean * self.seqs[r]) * (need - mean), -self.free[r], r))
        else:
            best = max(cand, key=lambda r: (self.free[r], -self.seqs[r], -r))
        self.free[best] -= need; self.used[best] += need; self.seqs[best] += 1
        self.placed[request_id] = (best, need)
        return best

    def release(self, request_id):
        r, need = self.placed.pop(request_id)
        self.free[r] += need; self.used[r] -= need; self.seqs[r] -= 1
        return r

    def owner(self, request_id):
        return self.placed[request_id][0]

    def refresh(self, dist, my_free_blocks, my_seqs):
        """Replaces the estimates by what every replica measured (rank order); a no-op without a process group."""
        if dist is None:
            self.free[0], self.seqs[0] = int(my_free_blocks), int(my_seqs)
            return
        got = [None] * self.world
        dist.all_gather_object(got, (int(my_free_blocks), int(my_seqs)))
        self.free = [g[0] for g in got]; self.seqs = [g[1] for g in got]


def gather_objects(dist, obj):
    """One picklable object per rank, in rank order, on every rank."""
    if dist is None:
        return [obj]
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj)
    return out


def rank_seeds(rank, base=0):
    """Distinct synthetic-data seeds per replica: (workload rng, weights, free-list shuffle, KV fill stride)."""
    return {"workload": base + 2 + rank, "weights": base + rank, "free_list": base + 3 + rank, "kv_fill": 1000 * rank}


GLOBAL_WORKLOAD_SEED = 2      # the one arrival stream every rank replays through the dispatcher


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
