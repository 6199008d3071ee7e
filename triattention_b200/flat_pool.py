"""Compaction for token-granular KV pools, with the entry point of the reference's SGLang backend.

SGLang keeps one ``[total_tokens, H, D]`` K tensor and one V tensor per layer and a ``req_to_token`` table that
maps a request's logical positions to pool slots (triattention/sglang/kv_compaction.py:282-404).  That is the paged
layout with a block size of one token, so the same CUDA kernel does the work: the request's ``req_to_token`` row
is its block table, read on the device without a host copy.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _native, ops


def compact_request_kv_in_place_per_head(
    k_buffers: List[torch.Tensor],
    v_buffers: List[torch.Tensor],
    req_to_token: torch.Tensor,
    req_pool_idx: int,
    keep_indices_per_head: torch.Tensor,
    effective_len: int,
    target_layers: Optional[List[int]] = None,
) -> int:
    """Move, per KV head, token ``keep_indices_per_head[h, i]`` of the request to its logical position ``i``.

    Same arguments, return value and errors as the reference (sglang/kv_compaction.py:282-404): ``k_buffers`` /
    ``v_buffers`` per-layer ``[total_tokens, H, D]`` bf16 tensors, ``req_to_token`` ``[max_reqs, max_context]`` int32,
    ``keep_indices_per_head`` ``[H, budget]`` ascending positions.  Returns the budget.  One kernel launch covers all
    target layers; validation costs one host synchronisation (the reference takes three).
    """
    if not k_buffers or len(k_buffers) != len(v_buffers):
        raise ValueError("k_buffers and v_buffers must be non-empty lists of equal length")
    dev = k_buffers[0].device
    keep = keep_indices_per_head.to(device=dev)
    H, budget = int(keep.shape[0]), int(keep.shape[1])
    if budget <= 0:
        return 0
    if budget > effective_len:
        raise ValueError(f"budget ({budget}) exceeds effective_len ({effective_len})")
    flags = torch.stack([(keep < 0).any(), (keep >= effective_len).any(),
                         (keep[:, 1:] <= keep[:, :-1]).any() if budget > 1 else torch.zeros((), dtype=torch.bool, device=dev)])
    neg, high, unsorted = (bool(x) for x in flags.tolist())
    if neg:
        raise IndexError("keep_indices_per_head contains negative values")
    if high:
        raise IndexError(f"keep_indices_per_head max >= effective_len ({effective_len})")
    if unsorted:
        raise ValueError("Each row of keep_indices_per_head must be sorted ascending to preserve original token order")
    layers = list(range(len(k_buffers))) if target_layers is None else [int(l) for l in target_layers]
    k0 = k_buffers[layers[0]]
    if k0.dtype != torch.bfloat16 or k0.ndim != 3 or k0.stride(2) != 1:
        raise ValueError("KV pool tensors must be [total_tokens, H, D] bf16 with a contiguous last axis")
    for l in layers:
        for t in (k_buffers[l], v_buffers[l]):
            if t.shape != k0.shape or t.stride() != k0.stride() or t.data_ptr() % 16:
                raise ValueError("all pool tensors must share shape and strides and be 16-byte aligned")
    view = ops.PagedCacheView(
        k_ptrs=torch.tensor([k_buffers[l].data_ptr() for l in layers], dtype=torch.int64, device=dev),
        v_ptrs=torch.tensor([v_buffers[l].data_ptr() for l in layers], dtype=torch.int64, device=dev),
        num_layers=len(layers), num_blocks=int(k0.shape[0]), block_size=1, num_kv_heads=int(k0.shape[1]),
        head_dim=int(k0.shape[2]), block_stride=int(k0.stride(0)), token_stride=int(k0.stride(0)),
        head_stride=int(k0.stride(1)), device=dev, dtype=k0.dtype)
    if H != view.num_kv_heads:
        raise ValueError(f"keep_indices_per_head has {H} rows, the pool has {view.num_kv_heads} KV heads")
    row = req_to_token[int(req_pool_idx)]
    if row.dtype != torch.int32 or not row.is_contiguous() or row.device != dev:
        row = row.to(device=dev, dtype=torch.int32).contiguous()
    slots = row[:effective_len].view(1, effective_len)
    layout = view.layout(1, 1, effective_len)
    meta = torch.tensor([effective_len, budget, 0], dtype=torch.int32, device=dev)
    ops.compact_paged(view, layout, slots, meta[0:1], keep.to(torch.int32).contiguous(), (0, 0, budget), meta[1:2], meta[2:3])
    return budget
