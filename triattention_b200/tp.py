"""Tensor-parallel sharding of the compression path.

Under tensor parallelism the KV cache shards by KV head: rank ``r`` of ``tp`` owns KV heads
``[r*Hkv/tp, (r+1)*Hkv/tp)`` and the query-head statistics rows ``[r*Hq/tp, (r+1)*Hq/tp)`` of every layer
(the slicing the reference's SGLang path applies, sglang/scoring_utils.py:112-131; its vLLM path has no rank
awareness).  Scores, moments, group max, layer mean, top-k and compaction are all per KV head, so the default
per-head mode needs no communication.

Only the layer-shared keep set (one keep list for all heads = top-k of the max over heads,
selector_hf.py:636-637) spans ranks: every rank reduces its local heads and the fp32 ``[L * B, t_pad]`` rows
are combined by MAX.  When the layers divide over the ranks each rank finishes the rows of its share of the
layers only: the finalize kernel stores every row straight into the owner's receive slot over NVLink
(:class:`PeerRowExchange`, symmetric memory, plain peer stores), the owner folds the slots, runs the top-k on
its rows, and an all-gather of the keep indices completes the step; without symmetric memory a NCCL
reduce-scatter(MAX) moves the rows instead (half the bytes of an all-reduce on the wire and 1/N of the
selection work per rank either way).  Otherwise one all-reduce(MAX) makes the rows global and the
deterministic top-k yields identical keep sets everywhere.
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



# ------------------------------------------------------------------------------------------------ peer-store exchange
class PeerRowExchange:
    """Receive buffers for the scattered form of the layer-shared exchange.

    Every rank owns ``rows_per_rank`` consecutive score rows and holds ``[world, rows_per_rank, t_pad]`` fp32 receive
    slots in symmetric memory (``torch.distributed._symmetric_memory``: the same allocation on every rank, mapped
    into every peer's address space; multicast binding is switched off - plain peer stores are all that is used).
    ``ptrs`` is the int64 device tensor of the ranks' buffer addresses that ``ops.finalize_scores_scatter`` stores
    through; ``barrier`` is a one-element NCCL all-reduce: when it has completed on this rank, every rank's finalize
    has, and with it all stores into this rank's slots.  The buffer is sized for the largest step seen so far.
    """

    def __init__(self, capacity_floats: int, device: torch.device, group=None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.capacity = int(capacity_floats)
        self._flat = symm_mem.empty(self.capacity, dtype=torch.float32, device=device)
        self._handle = symm_mem.rendezvous(self._flat, self.group)
        ptrs = [int(p) for p in self._handle.buffer_ptrs]
        if len(ptrs) != self.world or any(p == 0 for p in ptrs) or ptrs[self.rank] != self._flat.data_ptr():
            raise RuntimeError("symmetric memory did not return one mapped buffer per rank")
        self.ptrs = torch.tensor(ptrs, dtype=torch.int64, device=device)
        try:  # informational: with the switch above no multicast object should be bound to the buffers
            self.multicast_bound = int(getattr(self._handle, "multicast_ptr", 0) or 0) != 0
        except Exception:
            self.multicast_bound = None
        self._folded = torch.empty(self.capacity // self.world, dtype=torch.float32, device=device)
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def views(self, rows_per_rank: int, t_pad: int):
        """``(slots [world, rows_per_rank, t_pad], folded [rows_per_rank, t_pad])`` over the front of the buffers."""
        n = rows_per_rank * t_pad
        return (self._flat[: self.world * n].view(self.world, rows_per_rank, t_pad),
                self._folded[:n].view(rows_per_rank, t_pad))

    def barrier(self) -> None:
        dist.all_reduce(self._token, group=self.group)


_PEER_EXCHANGES: dict = {}


def peer_row_exchange(rows_per_rank: int, t_pad: int, device: torch.device, group=None) -> Optional[PeerRowExchange]:
    """Exchange buffers large enough for this step (made, or grown, collectively: every rank asks with the same
    shape in the same step), or None where symmetric memory cannot be set up - then the NCCL reduce-scatter serves.
    ``TRIATTN_TP_PEER_STORES=0`` switches the peer-store form off."""
    import os

    if os.environ.get("TRIATTN_TP_PEER_STORES", "1").strip().lower() in {"0", "false", "no", "off"}:
        return None
    if not (dist.is_available() and dist.is_initialized()) or torch.device(device).type != "cuda":
        return None
    if dist.get_backend(group) != "nccl":
        return None
    world = dist.get_world_size(group)
    need = world * int(rows_per_rank) * int(t_pad)
    key = (id(group), str(device))
    have = _PEER_EXCHANGES.get(key, "unset")
    if have is None or (have != "unset" and have.capacity >= need):
        return have
    try:
        made: Optional[PeerRowExchange] = PeerRowExchange(need, device, group)
    except Exception as exc:  # no permission for the handle exchange, an older torch, no peer access ...
        import logging
        logging.getLogger(__name__).warning("peer-store exchange unavailable (%s: %s); using NCCL reduce-scatter",
                                            type(exc).__name__, str(exc)[:200])
        made = None
    # all ranks take the same road: one rank without the buffers sends everybody to NCCL, for good
    ok = torch.tensor([1 if made is not None else 0], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    _PEER_EXCHANGES[key] = made if int(ok.item()) == 1 else None
    return _PEER_EXCHANGES[key]
