"""CPU restatement of the reference paged-cache primitives.  Test infrastructure only.

Follows ``triattention/vllm/runtime/kv_compaction.py`` (axis split :94-117,
dense gather :292-352, shared compaction :355-458, per-head compaction
:461-546, fallback keep builder :60-91) and
``triattention/vllm/runtime/layout_engine.py:209-227`` (tail-block truncation).
"""
from __future__ import annotations

from typing import Sequence

import torch


def split_kv_axes(kv_cache: torch.Tensor, kv_axis: int | None = None):
    """(key_cache, value_cache) views ``[nb, bs, H, D]`` of a 5-D paged cache (kv_compaction.py:94-117).

    ``kv_axis`` plays the role of the reference's registered layout hint when
    both leading dims have size 2.
    """
    if kv_cache.ndim != 5:
        raise ValueError(f"Unsupported kv_cache ndim={kv_cache.ndim}, expect 5")
    d0 = int(kv_cache.shape[0]) == 2
    d1 = int(kv_cache.shape[1]) == 2
    if d0 and d1:
        if kv_axis is None:
            raise ValueError("Ambiguous KV layout for compaction")
        d0, d1 = kv_axis == 0, kv_axis == 1
    if d0:
        return kv_cache[0], kv_cache[1]
    if d1:
        return kv_cache[:, 0], kv_cache[:, 1]
    raise ValueError("Unsupported KV layout for compaction: expected a dimension with size 2")


def _slots(block_ids: Sequence[int] | torch.Tensor, block_size: int, token_idx: torch.Tensor):
    """token index -> (physical block, offset) (kv_compaction.py:139-157)."""
    bt = torch.as_tensor(block_ids, dtype=torch.long)
    lb = torch.div(token_idx, block_size, rounding_mode="floor")
    if lb.numel() > 0 and int(lb.max()) >= int(bt.numel()):
        raise IndexError(
            f"token indices require block_idx={int(lb.max())}, but only {int(bt.numel())} blocks exist"
        )
    return bt[lb], torch.remainder(token_idx, block_size)


def gather_request_k_dense(kv_cache, block_ids, block_size, total_tokens, kv_axis=None) -> torch.Tensor:
    """Dense K ``[1, H, T, D]`` of one request (kv_compaction.py:292-319)."""
    if total_tokens <= 0:
        raise ValueError(f"total_tokens must be > 0, got {total_tokens}")
    key_cache, _ = split_kv_axes(kv_cache, kv_axis)
    blk, off = _slots(block_ids, block_size, torch.arange(total_tokens, dtype=torch.long))
    return key_cache[blk, off].transpose(0, 1).unsqueeze(0)


def compact_per_head(
    kv_cache: torch.Tensor,
    block_ids,
    block_size: int,
    keep_per_head: torch.Tensor,
    total_tokens: int,
    preserve_dropped_tokens: bool = True,
    kv_axis: int | None = None,
) -> int:
    """In-place per-KV-head compaction (kv_compaction.py:461-546).

    Head ``h`` ends with tokens ``keep[h, :]`` in slots ``0..k-1`` and, when
    ``preserve_dropped_tokens``, every other token in ascending order in slots
    ``k..T-1``.  With ``preserve_dropped_tokens=False`` only the kept prefix is
    written (slots >= k keep their old content) - the contract the CUDA
    compaction implements by default; the reference's own fill-hole variant
    (:564-589) scrambles prefix order and is never used in production
    (layout_engine.py:71-80).
    """
    key_cache, value_cache = split_kv_axes(kv_cache, kv_axis)
    H = int(key_cache.shape[2])
    keep = torch.as_tensor(keep_per_head, dtype=torch.long)
    if keep.ndim != 2:
        raise ValueError(f"keep_token_indices_per_head must be 2D, got shape={tuple(keep.shape)}")
    if int(keep.shape[0]) != H:
        raise ValueError(f"head count mismatch: expected {H}, got {int(keep.shape[0])}")
    k = int(keep.shape[1])
    if k <= 0:
        return 0
    if int(keep.min()) < 0 or int(keep.max()) >= total_tokens:
        raise IndexError(
            f"keep token index out of range: min={int(keep.min())}, max={int(keep.max())}, "
            f"expected [0, {total_tokens})"
        )
    srt = torch.sort(keep, dim=1).values
    if k > 1 and bool((srt[:, 1:] == srt[:, :-1]).any()):
        raise ValueError("per-head keep indices must not contain duplicates")
    if torch.equal(keep, torch.arange(k).unsqueeze(0).expand(H, -1)):
        return k
    if preserve_dropped_tokens:
        mask = torch.ones((H, total_tokens), dtype=torch.bool)
        mask.scatter_(1, keep, False)
        allt = torch.arange(total_tokens).unsqueeze(0).expand(H, -1)
        tail = allt[mask].view(H, total_tokens - k)
        perm = torch.cat([keep, tail], dim=1)
        n_dst = total_tokens
    else:
        perm = keep
        n_dst = k
    sb, so = _slots(block_ids, block_size, perm)
    hidx = torch.arange(H).unsqueeze(1)
    gk = key_cache[sb, so, hidx].clone()
    gv = value_cache[sb, so, hidx].clone()
    db, do = _slots(block_ids, block_size, torch.arange(n_dst, dtype=torch.long))
    key_cache[db, do] = gk.permute(1, 0, 2).contiguous()
    value_cache[db, do] = gv.permute(1, 0, 2).contiguous()
    return k


def compact_shared(
    kv_cache: torch.Tensor,
    block_ids,
    block_size: int,
    keep: torch.Tensor,
    total_tokens: int,
    preserve_dropped_tokens: bool = True,
    kv_axis: int | None = None,
) -> int:
    """In-place compaction with one keep list for all heads (kv_compaction.py:355-439)."""
    key_cache, value_cache = split_kv_axes(kv_cache, kv_axis)
    keep = torch.as_tensor(keep, dtype=torch.long).flatten()
    k = int(keep.numel())
    if k == 0:
        return 0
    if int(keep.min()) < 0 or int(keep.max()) >= total_tokens:
        raise IndexError(
            f"keep token index out of range: min={int(keep.min())}, max={int(keep.max())}, "
            f"expected [0, {total_tokens})"
        )
    if int(torch.unique(keep).numel()) != k:
        raise ValueError("keep_token_indices must not contain duplicates")
    if k >= total_tokens or torch.equal(keep, torch.arange(k)):
        return k
    if preserve_dropped_tokens:
        mask = torch.ones(total_tokens, dtype=torch.bool)
        mask[keep] = False
        perm = torch.cat([keep, torch.arange(total_tokens)[mask]])
        n_dst = total_tokens
    else:
        perm = keep
        n_dst = k
    sb, so = _slots(block_ids, block_size, perm)
    gk = key_cache[sb, so].clone()
    gv = value_cache[sb, so].clone()
    db, do = _slots(block_ids, block_size, torch.arange(n_dst, dtype=torch.long))
    key_cache[db, do] = gk
    value_cache[db, do] = gv
    return k


def truncate_tail_blocks(block_ids: Sequence[int], cache_len_after: int, block_size: int):
    """(kept, removed) block-id lists after compaction (layout_engine.py:209-227)."""
    required = 0 if cache_len_after <= 0 else (cache_len_after + block_size - 1) // block_size
    ids = [int(b) for b in block_ids]
    return ids[:required], ids[required:]


def fallback_keep_indices(total_tokens, kv_budget, prefill_len, protect_prefill, include_prefill_in_budget=True):
    """Recency keep list used when no selector is available (kv_compaction.py:60-91)."""
    budget = kv_budget
    if protect_prefill and not include_prefill_in_budget:
        budget += max(prefill_len, 0)
    budget = min(total_tokens, budget)
    if total_tokens <= budget:
        return list(range(total_tokens))
    if protect_prefill:
        if include_prefill_in_budget and prefill_len > budget:
            return None
        tail_need = max(0, budget - prefill_len)
        tail_start = max(prefill_len, total_tokens - tail_need)
        return list(range(prefill_len)) + list(range(tail_start, total_tokens))
    return list(range(max(0, total_tokens - budget), total_tokens))
