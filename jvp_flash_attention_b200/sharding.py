"""(batch x head) sharding over ranks, one process per GPU.

Every (batch, head) pair of an attention call is independent in forward, backward and the
Hessian-vector product, so a rank only needs its own contiguous slice of the flattened batch*head
axis and the data path has no collective.  ``gather_heads`` exists for verification only: it
brings the shards of a result back together (NCCL over NVLink on GPUs, gloo on CPUs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .workloads import shard_range


def local_heads(total_heads: int, group=None) -> tuple[int, int]:
    """[start, stop) of the flattened (batch*head) units owned by the calling rank."""
    if dist.is_available() and dist.is_initialized():
        return shard_range(total_heads, dist.get_rank(group), dist.get_world_size(group))
    return 0, total_heads


def gather_heads(shard: torch.Tensor, total_heads: int, group=None) -> torch.Tensor:
    """All-gathers per-rank shards of shape (n_local, ...) into (total_heads, ...) on every rank.

    Shards may differ in length by one (see ``shard_range``); they are padded to the longest for
    the collective and trimmed afterwards.  Without an initialised process group the shard is
    returned unchanged."""
    if not (dist.is_available() and dist.is_initialized()):
        return shard
    world = dist.get_world_size(group)
    sizes = [shard_range(total_heads, r, world) for r in range(world)]
    longest = max(hi - lo for lo, hi in sizes)
    pad = torch.zeros((longest,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    pad[: shard.shape[0]] = shard
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, sizes)], dim=0)
