"""Effective-length overrides for the forward inputs after a compaction, with the call signatures of the
reference's runtime/input_patch_ops.py (:66-215), on one CUDA kernel (``triattn_apply_effective_overrides``).

A compressed request attends over ``effective_base + query_len`` cached tokens instead of its absolute length;
the sparse per-request maps of the reference (dict: request-state row -> value) become dense int32 arrays over
request-state rows, the kernel handles the whole batch in one launch, and the "every key must be present in the
batch" checks of the reference are answered from counters the kernel fills.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from . import _native
from .ops import _ptr, _require_cuda, _stream


def _i32(t: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
    t = t if n is None else t[:n]
    return t.to(dtype=torch.int32).contiguous()


def _dense(values_by_row: dict, fill: int, device) -> torch.Tensor:
    size = max(int(k) for k in values_by_row) + 1
    host = np.full(size, fill, dtype=np.int32)
    for k, v in values_by_row.items():
        host[int(k)] = int(v)
    return torch.from_numpy(host).to(device)


def _launch(idx, qsl, num_reqs, base, delta, seq_lens, positions, positions_out, apply: bool) -> torch.Tensor:
    lib = _native.load()
    counters = torch.empty(4, dtype=torch.int32, device=idx.device)
    rows = int(base.numel()) if base is not None else (int(delta.numel()) if delta is not None else 0)
    _native.check(lib.triattn_apply_effective_overrides(
        _ptr(idx), _ptr(qsl), int(num_reqs), _ptr(base), _ptr(delta), rows, _ptr(seq_lens), _ptr(positions),
        _ptr(positions_out), int(positions.numel()) if positions is not None else 0, _ptr(counters), 1 if apply else 0,
        _stream()), "apply_effective_overrides")
    return counters


def overwrite_seq_lens_from_effective_lengths(*, idx_mapping: torch.Tensor, query_start_loc: torch.Tensor,
                                              effective_num_computed_tokens: torch.Tensor, seq_lens: torch.Tensor) -> None:
    """``seq_lens[r] = effective_num_computed_tokens[idx_mapping[r]] + query_len[r]`` for every batch entry."""
    num_reqs = int(idx_mapping.shape[0])
    if num_reqs <= 0:
        return
    _require_cuda(seq_lens, "seq_lens")
    dev = seq_lens.device
    work = seq_lens if seq_lens.dtype == torch.int32 and seq_lens.is_contiguous() else _i32(seq_lens)
    _launch(_i32(idx_mapping.to(dev)), _i32(query_start_loc.to(dev), num_reqs + 1), num_reqs,
            _i32(effective_num_computed_tokens.to(dev)), None, work, None, None, True)
    if work is not seq_lens:
        seq_lens.copy_(work)


def overwrite_seq_lens_from_effective_base_map(*, idx_mapping: torch.Tensor, query_start_loc: torch.Tensor,
                                               effective_base_by_req_idx: dict, seq_lens: torch.Tensor,
                                               effective_base_lookup_tensors=None) -> bool:
    """Overwrite the entries whose request-state row has an effective base; False (nothing written) unless every
    key of the map belongs to exactly one batch entry."""
    num_reqs = int(idx_mapping.shape[0])
    if num_reqs <= 0 or not effective_base_by_req_idx:
        return False
    _require_cuda(seq_lens, "seq_lens")
    dev = seq_lens.device
    idx, qsl = _i32(idx_mapping.to(dev)), _i32(query_start_loc.to(dev), num_reqs + 1)
    base = _dense(effective_base_by_req_idx, -1, dev)
    matched = int(_launch(idx, qsl, num_reqs, base, None, None, None, None, False)[0].item())
    if matched == 0 or matched != len(effective_base_by_req_idx):
        return False
    work = seq_lens if seq_lens.dtype == torch.int32 and seq_lens.is_contiguous() else _i32(seq_lens)
    _launch(idx, qsl, num_reqs, base, None, work, None, None, True)
    if work is not seq_lens:
        seq_lens.copy_(work)
    return True


def shift_positions_from_sparse_deltas(*, idx_mapping: torch.Tensor, query_start_loc: torch.Tensor,
                                       positions: torch.Tensor, pos_delta_by_req_idx: dict,
                                       pos_delta_lookup_tensors=None) -> Optional[torch.Tensor]:
    """A copy of ``positions`` with each request's query tokens shifted by its delta; None when the reference
    would decline (a key without a batch entry, decreasing ``query_start_loc``, no non-zero delta, no query
    tokens, or a shifted segment outside the buffer)."""
    num_reqs = int(idx_mapping.shape[0])
    if num_reqs <= 0 or not pos_delta_by_req_idx:
        return None
    _require_cuda(positions, "positions")
    dev = positions.device
    idx, qsl = _i32(idx_mapping.to(dev)), _i32(query_start_loc.to(dev), num_reqs + 1)
    # membership is counted on a copy of the map in which every key is marked (a delta may be zero)
    present = _dense({k: 1 for k in pos_delta_by_req_idx}, -1, dev)
    delta = _dense(pos_delta_by_req_idx, 0, dev)
    pos64 = positions.to(dtype=torch.int64).contiguous()
    out = torch.empty_like(pos64)
    c_members = _launch(idx, qsl, num_reqs, present, None, None, None, None, False)
    c_apply = _launch(idx, qsl, num_reqs, None, delta, None, pos64, out, True)
    members = int(c_members[0].item())
    changed, decreasing, outside = (int(x) for x in c_apply[1:4].tolist())
    if members != len(pos_delta_by_req_idx) or decreasing or changed == 0:
        return None
    q_host = qsl[[0, num_reqs]].tolist()
    total = q_host[1] - q_host[0]
    if total <= 0:
        return None
    if not (q_host[0] == 0 and total <= int(pos64.numel())):
        # explicit-index path of the reference: the changed rows need query tokens, all inside the buffer
        q_all = qsl.tolist()
        rows = idx.tolist()
        changed_lens = [q_all[r + 1] - q_all[r] for r in range(num_reqs)
                        if pos_delta_by_req_idx.get(rows[r], 0) != 0]
        if sum(changed_lens) == 0:
            return None
        for r in range(num_reqs):
            if pos_delta_by_req_idx.get(rows[r], 0) != 0 and q_all[r + 1] > q_all[r] and \
                    (q_all[r] < 0 or q_all[r + 1] > int(pos64.numel())):
                return None
    return out.to(dtype=positions.dtype)
