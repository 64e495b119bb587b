"""Sharding of independent kernels / queries across the GPUs of one box.

Every (kernel, destination) pair and every MLP query is independent, so ranks
take contiguous shards, run the same kernels on them and exchange nothing but
totals: one all-reduce (sums per destination) or one all-gather (per-iteration
totals) per batch, a few KB over NCCL.  The reference has no counterpart: its
prediction path is a single host thread.
"""
import os

import torch
import torch.distributed as dist


def env_rank_world():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init(backend=None):
    """Joins the process group described by RANK / WORLD_SIZE / MASTER_* (one
    process per GPU).  NCCL when CUDA is present, gloo otherwise."""
    rank, world = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, world


_host_group = None


def host_group():
    """A gloo group over the same ranks, for waits that should not occupy the GPUs: a rank
    blocked in a NCCL barrier spins on its GPU, a rank blocked here sleeps on a socket."""
    global _host_group
    if _host_group is None and dist.is_initialized() and dist.get_world_size() > 1:
        _host_group = dist.new_group(backend="gloo")
    return _host_group


def host_barrier():
    """Barrier over the host group (no-op on one rank).  All ranks must call it."""
    g = host_group()
    if g is not None:
        dist.barrier(group=g)


def shard_bounds(n, rank, world):
    """Contiguous near-equal shards: the first n % world ranks hold one more item."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_bounds_aligned(n, rank, world, align=4):
    """As shard_bounds, but every boundary except the last is a multiple of
    `align`, so each shard keeps the wide (16-byte) load path."""
    blocks = (n + align - 1) // align
    lo, hi = shard_bounds(blocks, rank, world)
    return min(lo * align, n), min(hi * align, n)


def allreduce_sum_(totals):
    """In-place sum over ranks of a tensor of totals (no-op on one rank)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
    return totals


def allgather_rows(local_rows, world=None):
    """Concatenates per-rank [n_r, D] blocks of per-iteration totals in rank order."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return local_rows
    world = dist.get_world_size()
    sizes = [torch.zeros(1, dtype=torch.int64, device=local_rows.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([local_rows.shape[0]], dtype=torch.int64, device=local_rows.device))
    n_max = int(max(int(s.item()) for s in sizes))
    pad = torch.zeros((n_max,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    pad[:local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[:int(s.item())] for p, s in zip(parts, sizes)], dim=0)


def sharded_totals(n_items, compute_totals, rank=None, world=None, align=4):
    """Runs `compute_totals(lo, hi) -> tensor of sums` on this rank's shard of
    n_items and returns the totals summed over all ranks."""
    if rank is None or world is None:
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
    lo, hi = shard_bounds_aligned(n_items, rank, world, align)
    return allreduce_sum_(compute_totals(lo, hi))
