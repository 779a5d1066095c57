"""(batch x head) sharding of the hot path across the GPUs of one box.

Every (batch, head) pair is independent in the forward and in the backward (the reference marks those grid
axes "parallel", flex_attention_kernel.py:184-186), so the path shards with no exchange: rank r owns a
contiguous range of the flattened batch*head index.  Collectives appear only around it: a gather of the
outputs for checking.  Works with any torch.distributed backend (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_bounds(units: int, world: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of the units owned by `rank`: contiguous, sizes differ by at most one, covers 0..units."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch_heads(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Slice of a [B, H, S, D] (or [B, H, S]) tensor owned by `rank`, as [1, units, ...] (units = the rank's
    share of B*H), contiguous: a valid input of the entry points with batch = 1, heads = units."""
    B, H = t.shape[:2]
    lo, hi = shard_bounds(B * H, world, rank)
    return t.reshape(B * H, *t.shape[2:])[lo:hi].unsqueeze(0).contiguous()


def gather_batch_heads(shard: torch.Tensor, batch: int, heads: int, group=None) -> torch.Tensor:
    """Inverse of shard_batch_heads on every rank: all-gathers the [1, units_r, ...] shards and returns the full
    [batch, heads, ...] tensor.  Used for verification only; shards may differ in size by one unit."""
    world = dist.get_world_size(group)
    sizes = [shard_bounds(batch * heads, world, r) for r in range(world)]
    max_units = max(hi - lo for lo, hi in sizes)
    pad = torch.zeros((max_units, *shard.shape[2:]), dtype=shard.dtype, device=shard.device)
    pad[: shard.shape[1]] = shard[0]
    parts: List[torch.Tensor] = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    full = torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, sizes)], dim=0)
    return full.reshape(batch, heads, *shard.shape[2:])
