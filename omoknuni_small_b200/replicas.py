"""Multi-GPU plumbing: independent replicas, no collective on the data path.

Each GPU runs its own game shard (its own trees, its own weight replica, its
own leaf batches); nothing on the hot path crosses GPUs.  What does cross:
a barrier on both sides of a timed region, the max over ranks of the device
times, and — after the timed region — the sum of the per-GPU counters
(evaluations, batches, selections, ...).  The reference has no multi-GPU path
at all; its unit of parallelism is one engine per game thread
(reference src/selfplay/self_play_manager.cpp:360-376), which is what a rank
is here.

The functions take a torch.distributed module (or None for a single process)
so that they run unchanged over NCCL on GPUs and over gloo on CPUs.
"""
import os


def rank_info():
    """(rank, world_size, local_rank) from the torchrun environment."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def shard_seed(base_seed, rank):
    """Seed of a rank's shard of synthetic games / trees: shards differ across
    ranks and do not depend on the world size, so a shard's results are the
    same whether 1 or 8 GPUs run."""
    return int(base_seed) + 7919 * int(rank)


def shard_range(n_items, rank, world):
    """Contiguous [lo, hi) slice of n_items for this rank (strong-scaling split)."""
    base, extra = divmod(int(n_items), int(world))
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def max_over_ranks(dist, values, device="cpu"):
    """Element-wise max over ranks of a list of floats (device times in ms)."""
    if dist is None:
        return [float(v) for v in values]
    import torch
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def sum_counters(dist, counters, device="cpu"):
    """Sum of per-rank counter dicts (the end-of-run reduction)."""
    keys = sorted(counters)
    if dist is None:
        return {k: int(counters[k]) for k in keys}
    import torch
    t = torch.tensor([int(counters[k]) for k in keys], dtype=torch.int64, device=device)
    dist.all_reduce(t)
    return dict(zip(keys, t.tolist()))


def aggregate_throughput(units_per_rank_per_step, steps, world, max_ms):
    """Whole-job throughput: the units all ranks processed / the slowest rank's time."""
    return world * units_per_rank_per_step * steps / (max_ms * 1e-3)
