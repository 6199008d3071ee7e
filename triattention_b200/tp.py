"""Tensor-parallel sharding of the compression path.

Under tensor parallelism the KV cache shards by KV head: rank ``r`` of ``tp`` owns KV heads
``[r*Hkv/tp, (r+1)*Hkv/tp)`` and the query-head statistics rows ``[r*Hq/tp, (r+1)*Hq/tp)`` of every layer
(the slicing the reference's SGLang path applies, sglang/scoring_utils.py:112-131; its vLLM path has no rank
awareness).  Scores, moments, group max, layer mean, top-k and compaction are all per KV head, so the default
per-head mode needs no communication.

Only the layer-shared keep set (one keep list for all heads = top-k of the max over heads,
selector_hf.py:636-637) spans ranks: every rank reduces its local heads, one all-reduce(MAX) of the fp32
``[B, t_pad]`` rows makes them global, and the deterministic top-k then yields identical keep sets on every
rank without a broadcast.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def head_range(num_heads: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Half-open range of heads owned by ``rank``; ``num_heads`` must divide evenly."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    if num_heads % world_size != 0:
        raise ValueError(f"{num_heads} heads do not shard evenly over {world_size} ranks")
    per = num_heads // world_size
    return rank * per, (rank + 1) * per


def shard_stats(stats: ops.DeviceStats, rank: int, world_size: int) -> ops.DeviceStats:
    """Statistics rows of the query heads whose KV heads live on ``rank``."""
    lo, hi = head_range(stats.num_heads, rank, world_size)
    return stats.slice_heads(lo, hi)


def allreduce_shared_scores(local_head_max: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """In-place all-reduce(MAX) of per-rank ``max over local heads`` score rows (``[..., t_pad]`` fp32).

    +inf guard entries and the -inf padding beyond each request's length are preserved by MAX.
    Returns its argument; a no-op when torch.distributed is not initialised or the group has one rank.
    """
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(local_head_max, op=dist.ReduceOp.MAX, group=group)
    return local_head_max
