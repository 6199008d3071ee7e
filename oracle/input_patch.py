"""CPU checker (test infrastructure, not a product path) for the effective-length overrides applied to the
forward inputs after a compaction.  numpy restatement of triattention/vllm/runtime/input_patch_ops.py:

* ``seq_lens_from_effective_lengths``  - overwrite_seq_lens_from_effective_lengths (:66-83)
* ``seq_lens_from_effective_base_map`` - overwrite_seq_lens_from_effective_base_map (:86-124)
* ``shift_positions_from_sparse_deltas`` (:127-215)

Pinned by tests/golden/input_patch_cases.npz (outputs of those functions themselves).
"""
from __future__ import annotations

from typing import Optional

import numpy as np


def seq_lens_from_effective_lengths(idx_mapping, query_start_loc, effective_num_computed_tokens, seq_lens) -> np.ndarray:
    out = np.array(seq_lens, copy=True)
    n = len(idx_mapping)
    if n <= 0:
        return out
    q = np.asarray(query_start_loc, dtype=np.int64)
    base = np.asarray(effective_num_computed_tokens, dtype=np.int64)[np.asarray(idx_mapping, dtype=np.int64)]
    out[:n] = (base + (q[1:n + 1] - q[:n])).astype(out.dtype)
    return out


def seq_lens_from_effective_base_map(idx_mapping, query_start_loc, base_by_row: dict, seq_lens):
    """(applied, seq_lens): applied only if every key of the map is the row of exactly the matched batch entries."""
    out = np.array(seq_lens, copy=True)
    n = len(idx_mapping)
    if n <= 0 or not base_by_row:
        return False, out
    rows = [int(r) for r in idx_mapping]
    hits = [r for r in range(n) if rows[r] in base_by_row]
    if not hits or len(hits) != len(base_by_row):
        return False, out
    q = np.asarray(query_start_loc, dtype=np.int64)
    for r in hits:
        out[r] = base_by_row[rows[r]] + int(q[r + 1] - q[r])
    return True, out


def shift_positions_from_sparse_deltas(idx_mapping, query_start_loc, positions, delta_by_row: dict) -> Optional[np.ndarray]:
    n = len(idx_mapping)
    if n <= 0 or not delta_by_row:
        return None
    rows = [int(r) for r in idx_mapping]
    hits = [r for r in range(n) if rows[r] in delta_by_row]
    if len(hits) != len(delta_by_row):
        return None
    q = np.asarray(query_start_loc, dtype=np.int64)
    if np.any(q[1:n + 1] < q[:n]):
        return None
    if not any(delta_by_row[rows[r]] != 0 for r in hits):
        return None
    out = np.array(positions, copy=True)
    total = int(q[n] - q[0])
    if total == 0:
        return None
    changed = [r for r in hits if delta_by_row[rows[r]] != 0]
    if q[0] == 0 and total <= out.shape[0]:
        # contiguous packing from token 0: every segment lies inside the buffer
        for r in changed:
            out[q[r]:q[r + 1]] += delta_by_row[rows[r]]
        return out
    # explicit token indices of the changed rows, validated against the buffer
    if sum(int(q[r + 1] - q[r]) for r in changed) == 0:
        return None
    for r in changed:
        if q[r + 1] > q[r] and (q[r] < 0 or q[r + 1] > out.shape[0]):
            return None
    for r in changed:
        out[q[r]:q[r + 1]] += delta_by_row[rows[r]]
    return out
