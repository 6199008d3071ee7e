"""Block-table arithmetic after compaction (reference: runtime/layout_engine.py:24-27, :209-227)."""
from __future__ import annotations

from typing import Optional

from .plan_models import ReclaimGroup


def num_required_blocks(total_tokens: int, block_size: int) -> int:
    if total_tokens <= 0:
        return 0
    return (total_tokens + block_size - 1) // block_size


def truncate_tail_reclaim_group(*, gid: int, normalized_block_ids: list, cache_len_after: int,
                                block_size: int) -> tuple[list, list, Optional[ReclaimGroup]]:
    """Keep the first ceil(cache_len_after / block_size) block ids, hand the rest back."""
    required = num_required_blocks(cache_len_after, block_size)
    kept = list(normalized_block_ids[:required])
    removed = list(normalized_block_ids[required:])
    group = None
    if removed:
        group = ReclaimGroup(gid=gid, block_ids_before=list(normalized_block_ids), block_ids_after=kept,
                             block_ids_removed=removed)
    return kept, removed, group
