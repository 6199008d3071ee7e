"""Paged-cache primitives with the call signatures of the reference's runtime/kv_compaction.py.

``compact_request_kv_in_place`` / ``compact_request_kv_in_place_per_head`` validate their arguments
like the reference (same ``IndexError`` / ``ValueError`` cases, :375-397 and :477-510) and then run the
CUDA compaction kernel through the C ABI; there is no torch indexing path.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from . import _native, ops

_KV_LAYOUT_AXIS_HINTS: dict = {}


def _hint_key(kv_cache: torch.Tensor):
    return (int(kv_cache.data_ptr()), int(kv_cache.storage_offset()), tuple(int(x) for x in kv_cache.shape),
            tuple(int(x) for x in kv_cache.stride()), str(kv_cache.device))


def register_kv_layout_axis_hint(kv_cache: torch.Tensor, kv_axis: int) -> None:
    """Record which of the two size-2 leading axes is the K/V axis (kv_compaction.py:38-53)."""
    if kv_cache.ndim != 5:
        raise ValueError(f"Expected 5D kv_cache for layout hint, got ndim={kv_cache.ndim}")
    if kv_axis not in (0, 1):
        raise ValueError(f"kv_axis must be 0 or 1, got {kv_axis}")
    if int(kv_cache.shape[kv_axis]) != 2:
        raise ValueError(f"kv_axis={kv_axis} does not point to K/V dimension (shape={tuple(kv_cache.shape)})")
    _KV_LAYOUT_AXIS_HINTS[_hint_key(kv_cache)] = kv_axis


def clear_kv_layout_axis_hints_for_tests() -> None:
    _KV_LAYOUT_AXIS_HINTS.clear()


def kv_axis_hint(kv_cache: torch.Tensor) -> Optional[int]:
    return _KV_LAYOUT_AXIS_HINTS.get(_hint_key(kv_cache))


def _split_kv_axes(kv_cache: torch.Tensor):
    return ops.split_kv_axes(kv_cache, kv_axis_hint(kv_cache))


def build_keep_token_indices(total_tokens: int, kv_budget: int, prefill_len: int, protect_prefill: bool,
                             include_prefill_in_budget: bool = True):
    """Recency keep list used when no selector is available; None if the protected prefill cannot fit
    (kv_compaction.py:60-91)."""
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


def _block_table(block_ids, device) -> torch.Tensor:
    if isinstance(block_ids, torch.Tensor):
        return block_ids.to(device=device, dtype=torch.int32).reshape(1, -1).contiguous()
    return torch.as_tensor(list(block_ids), dtype=torch.int32, device=device).reshape(1, -1)


def gather_request_k_dense(kv_cache: torch.Tensor, block_ids, block_size: int, total_tokens: int) -> torch.Tensor:
    """Dense K ``[1, H, T, D]`` of one request (kv_compaction.py:292-319).  Debug/test helper: the scorer
    reads the paged cache directly and never needs this copy."""
    if total_tokens <= 0:
        raise ValueError(f"total_tokens must be > 0, got {total_tokens}")
    key_cache, _ = _split_kv_axes(kv_cache)
    bt = _block_table(block_ids, key_cache.device).long().flatten()
    tok = torch.arange(total_tokens, device=key_cache.device)
    lb = torch.div(tok, block_size, rounding_mode="floor")
    if int(lb.max()) >= int(bt.numel()):
        raise IndexError(f"token range requires block_idx={int(lb.max())}, but only {int(bt.numel())} blocks exist")
    return key_cache[bt[lb], tok % block_size].transpose(0, 1).unsqueeze(0)


def _run_compaction(kv_cache, block_ids, block_size, keep: torch.Tensor, head_stride: int, total_tokens: int,
                    preserve_dropped_tokens: bool) -> None:
    """One launch for one layer (``kv_cache`` a tensor) or for all layers of a group (a list of tensors)."""
    caches = list(kv_cache) if isinstance(kv_cache, (list, tuple)) else [kv_cache]
    kv_axis = kv_axis_hint(caches[0])
    view = ops.PagedCacheView.from_layers(caches, kv_axis=kv_axis)
    if view.block_size != int(block_size):
        raise ValueError(f"block_size={block_size} does not match the cache layout ({view.block_size})")
    dev = view.device
    bt = _block_table(block_ids, dev)
    need = (total_tokens + block_size - 1) // block_size
    if need > int(bt.shape[1]):
        raise IndexError(f"token indices require block_idx={need - 1}, but only {int(bt.shape[1])} blocks exist")
    k = int(keep.shape[-1])
    layout = view.layout(1, 1, int(bt.shape[1]))
    seq = torch.tensor([total_tokens], dtype=torch.int32, device=dev)
    kc = torch.tensor([k], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.compact_paged(view, layout, bt, seq, keep, (0, 0, head_stride), kc, status,
                      preserve_dropped=preserve_dropped_tokens, max_dropped_rows=max(total_tokens - k, 0))
    bits = int(status.item())
    if bits & _native.DEV_BAD_BLOCK_ID:
        raise IndexError("block id outside the cache")
    if bits & _native.DEV_BAD_KEEP_INDEX:
        raise IndexError("keep token index out of range or keep row not strictly ascending")
    if bits:
        raise RuntimeError(f"{_native.TRITON_SCORING_REQUIRED_MARKER}:compaction_device_status:{bits}")


def compact_request_kv_in_place(kv_cache: torch.Tensor, block_ids, block_size: int,
                                keep_token_indices: Iterable[int] | torch.Tensor, total_tokens: int,
                                preserve_dropped_tokens: bool = True) -> int:
    """Compact one request in place with one keep list for all heads; returns the keep count
    (kv_compaction.py:355-458).  Kept tokens land in slots ``0..k-1`` in the order given (ascending order
    is required here; the reference's selectors always produce it); with ``preserve_dropped_tokens`` the
    dropped tokens follow in ascending order, otherwise slots ``>= k`` keep their old content."""
    key_cache, _ = _split_kv_axes(kv_cache)
    dev = key_cache.device
    if isinstance(keep_token_indices, torch.Tensor):
        keep = keep_token_indices.to(device=dev, dtype=torch.long).flatten()
    else:
        keep = torch.as_tensor(list(keep_token_indices), device=dev, dtype=torch.long)
    k = int(keep.numel())
    if k == 0:
        return 0
    lo, hi = int(keep.min().item()), int(keep.max().item())
    if lo < 0 or hi >= total_tokens:
        raise IndexError(f"keep token index out of range: min={lo}, max={hi}, expected [0, {total_tokens})")
    if k > 1 and not bool((keep[1:] > keep[:-1]).all().item()):
        if int(torch.unique(keep).numel()) != k:
            raise ValueError("keep_token_indices must not contain duplicates")
        raise ValueError("keep_token_indices must be ascending")
    if k >= total_tokens:
        return k
    _run_compaction(kv_cache, block_ids, block_size, keep.to(torch.int32).contiguous(), 0, total_tokens,
                    preserve_dropped_tokens)
    return k


def compact_request_kv_in_place_per_head(kv_cache: torch.Tensor, block_ids, block_size: int,
                                         keep_token_indices_per_head, total_tokens: int,
                                         preserve_dropped_tokens: bool = True) -> int:
    """Compact one request in place with independent keep rows ``[Hkv, k]`` per KV head; returns ``k``
    (kv_compaction.py:461-599)."""
    key_cache, _ = _split_kv_axes(kv_cache)
    dev = key_cache.device
    H = int(key_cache.shape[2])
    if isinstance(keep_token_indices_per_head, torch.Tensor):
        keep = keep_token_indices_per_head.to(device=dev, dtype=torch.long)
    else:
        if not keep_token_indices_per_head:
            return 0
        keep = torch.as_tensor(keep_token_indices_per_head, device=dev, dtype=torch.long)
    if keep.ndim != 2:
        raise ValueError(f"keep_token_indices_per_head must be 2D, got shape={tuple(keep.shape)}")
    if int(keep.shape[0]) != H:
        raise ValueError(f"keep_token_indices_per_head head count mismatch: expected {H}, got {int(keep.shape[0])}")
    k = int(keep.shape[1])
    if k <= 0:
        return 0
    lo, hi = int(keep.min().item()), int(keep.max().item())
    if lo < 0 or hi >= total_tokens:
        raise IndexError(f"keep token index out of range: min={lo}, max={hi}, expected [0, {total_tokens})")
    if k > 1 and not bool((keep[:, 1:] > keep[:, :-1]).all().item()):
        srt = torch.sort(keep, dim=1).values
        if bool((srt[:, 1:] == srt[:, :-1]).any().item()):
            raise ValueError("per-head keep indices must not contain duplicates")
        raise ValueError("per-head keep indices must be ascending")
    _run_compaction(kv_cache, block_ids, block_size, keep.to(torch.int32).contiguous(), k, total_tokens,
                    preserve_dropped_tokens)
    return k


def compact_group_kv_in_place_per_head(kv_caches, block_ids, block_size: int, keep_token_indices_per_head,
                                       total_tokens: int, preserve_dropped_tokens: bool = False) -> int:
    """``compact_request_kv_in_place_per_head`` for every layer of a KV-cache group in one kernel launch.

    The default selection mode applies one keep set to all layers (selection_planner.py:183-193); the
    reference still compacts layer by layer (layout_engine.py:112-139).
    """
    caches = list(kv_caches)
    key_cache, _ = _split_kv_axes(caches[0])
    dev = key_cache.device
    H = int(key_cache.shape[2])
    keep = torch.as_tensor(keep_token_indices_per_head, device=dev).to(torch.long)
    if keep.ndim != 2:
        raise ValueError(f"keep_token_indices_per_head must be 2D, got shape={tuple(keep.shape)}")
    if int(keep.shape[0]) != H:
        raise ValueError(f"keep_token_indices_per_head head count mismatch: expected {H}, got {int(keep.shape[0])}")
    k = int(keep.shape[1])
    if k <= 0:
        return 0
    # range / order violations are caught on the device (status word) without reading the keep set back
    _run_compaction(caches, block_ids, block_size, keep.to(torch.int32).contiguous(), k, total_tokens,
                    preserve_dropped_tokens)
    return k
