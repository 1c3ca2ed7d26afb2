"""Data-parallel sharding of clips / streams over the GPUs of one box.

Clips (prefill) and streams (decode) are independent: attention never mixes batch rows
(src/fast_mimi/model.py:1896-1961) and KV state is per stream.  Each rank therefore owns a contiguous
block of units, weights are replicated, and there is no collective on the data path; results are
copied to pinned host memory per rank and concatenated there.
"""
from __future__ import annotations

import torch


def shard_bounds(n_units: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous block ``[lo, hi)`` of ``n_units`` owned by ``rank``; sizes differ by at most one."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad rank / world_size")
    base, extra = divmod(n_units, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard(t: torch.Tensor, world_size: int, rank: int, dim: int = 0) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[dim], world_size, rank)
    return t.narrow(dim, lo, hi - lo)


def gather_to_host(local: torch.Tensor, group=None) -> torch.Tensor | None:
    """Concatenate every rank's host tensor on rank 0 (off the hot path; uses the process group's own
    collective, gloo or nccl).  Returns the full tensor on rank 0 and None elsewhere."""
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local.cpu()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [None] * world
    dist.all_gather_object(sizes, tuple(local.shape), group=group)
    backend = dist.get_backend(group)
    dev = local.device if backend == "nccl" else torch.device("cpu")
    # Ranks may own blocks that differ by one unit: pad to the largest block, gather, trim.
    rows = max(s[0] for s in sizes)
    src = torch.zeros((rows, *local.shape[1:]), dtype=local.dtype, device=dev)
    src[: local.shape[0]] = local.to(dev)
    bufs = [torch.empty_like(src) for _ in range(world)]
    dist.all_gather(bufs, src, group=group)
    if rank != 0:
        return None
    return torch.cat([b[: s[0]].cpu() for b, s in zip(bufs, sizes)], dim=0)
