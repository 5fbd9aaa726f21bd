"""Host-side plumbing for running the path on several GPUs of one box.

Sequences (batch entries, heads) are independent, so the operator and the backbone shard by
batch with no collective on the data path: every rank owns a contiguous slice of the batch, runs
on its own GPU and keeps its outputs there.  The only exchanges are a barrier and a max-reduce of
the measured time, and an optional final gather of outputs for reporting or parity checks
(the reference's only multi-GPU inference path splits an image list by rank the same way,
tools/dota_submit.py:92-125).  Works with any torch.distributed backend (NCCL on GPUs, gloo in
the CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, stop) slice of `total` items owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Slowest rank's value (the time a multi-GPU step is charged)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def gather_batch(local: torch.Tensor, total: int, group=None) -> Optional[List[torch.Tensor]]:
    """Final gather of per-rank batch slices, outside any timed region.  Returns the slices in rank
    order on every rank and checks that they cover `total` items exactly, so that a rank that
    contributed a wrong or empty slice is reported instead of silently dropped."""
    if not (dist.is_available() and dist.is_initialized()):
        if local.shape[0] != total:
            raise RuntimeError(f"single process holds {local.shape[0]} of {total} items")
        return [local]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    sizes = [None] * world
    dist.all_gather_object(sizes, int(local.shape[0]), group=group)
    expected = [shard_range(total, r, world) for r in range(world)]
    bad = [r for r in range(world) if sizes[r] != expected[r][1] - expected[r][0]]
    if bad:
        raise RuntimeError(f"ranks {bad} hold {[sizes[r] for r in bad]} items, expected "
                           f"{[expected[r][1] - expected[r][0] for r in bad]}")
    parts = [torch.empty((sizes[r],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
             for r in range(world)]
    if len(set(sizes)) == 1:
        dist.all_gather(parts, local.contiguous(), group=group)
    else:
        _ragged_gather(parts, local, rank, group)
    return parts


def _ragged_gather(parts, local, rank, group):
    for r, buf in enumerate(parts):
        if r == rank:
            buf.copy_(local)
        dist.broadcast(buf, src=dist.get_global_rank(group, r) if group is not None else r, group=group)
