"""Tensor-parallel sharding of the compression path.

Under tensor parallelism the KV cache shards by KV head: rank ``r`` of ``tp`` owns KV heads
``[r*Hkv/tp, (r+1)*Hkv/tp)`` and the query-head statistics rows ``[r*Hq/tp, (r+1)*Hq/tp)`` of every layer
(the slicing the reference's SGLang path applies, sglang/scoring_utils.py:112-131; its vLLM path has no rank
awareness).  Scores, moments, group max, layer mean, top-k and compaction are all per KV head, so the default
per-head mode needs no communication.

Only the layer-shared keep set (one keep list for all heads = top-k of the max over heads,
selector_hf.py:636-637) spans ranks: every rank reduces its local heads and the fp32 ``[L * B, t_pad]`` rows
are combined by MAX.  When the layers divide over the ranks the exchange is a reduce-scatter (each rank
receives the finished rows of its share of the layers), a top-k on those rows only, and an all-gather of the
keep indices: half the bytes of an all-reduce on the wire and 1/N of the selection work per rank.  Otherwise
one all-reduce(MAX) makes the rows global and the deterministic top-k yields identical keep sets everywhere.
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


def _group_size(group) -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group)
    return 1


def can_scatter_rows(num_layers: int, group: Optional[dist.ProcessGroup] = None) -> bool:
    """True when the reduce-scatter form of the exchange applies: several ranks and whole layers per rank."""
    n = _group_size(group)
    return n > 1 and num_layers % n == 0


def reduce_scatter_shared_scores(rows: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """MAX-combine ``rows`` (``[R, t_pad]`` fp32, the same shape on every rank) and return this rank's
    ``R / world`` consecutive finished rows."""
    n = _group_size(group)
    if rows.shape[0] % n:
        raise ValueError(f"{rows.shape[0]} rows do not divide over {n} ranks")
    out = torch.empty((rows.shape[0] // n, rows.shape[1]), dtype=rows.dtype, device=rows.device)
    dist.reduce_scatter_tensor(out, rows.contiguous(), op=dist.ReduceOp.MAX, group=group)
    return out


def all_gather_keep(local_keep: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Concatenate the ranks' keep rows (``[R / world, keep_pitch]`` int32) in rank order: ``[R, keep_pitch]``."""
    n = _group_size(group)
    out = torch.empty((local_keep.shape[0] * n, local_keep.shape[1]), dtype=local_keep.dtype, device=local_keep.device)
    dist.all_gather_into_tensor(out, local_keep.contiguous(), group=group)
    return out

