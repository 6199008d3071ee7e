"""Records that travel through the hook pipeline - what to keep, which blocks a group gave back, and the result the
hook reports - with the dictionary layouts of the reference's ``runtime/plan_models.py:13-134`` (the scheduler and
the tests read those dictionaries, so keys and value types are fixed; everything else is this package's)."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Optional


# ------------------------------------------------------------------------------------------------ block reclaim
@dataclass(frozen=True)
class ReclaimGroup:
    """Block ids of one KV-cache group before the compaction, the kept prefix and the returned tail."""

    gid: int
    block_ids_before: list
    block_ids_after: list
    block_ids_removed: list

    def to_dict(self) -> dict:
        return {f.name: (list(v) if isinstance(v := getattr(self, f.name), list) else v)
                for f in dataclasses.fields(self)}


@dataclass(frozen=True)
class ReclaimEvent:
    mode: str      # "truncate_tail"
    groups: list   # of ReclaimGroup

    def reclaimed_block_count(self) -> int:
        return sum(map(len, (g.block_ids_removed for g in self.groups)))

    def to_dict(self) -> dict:
        return dict(mode=self.mode, groups=[g.to_dict() for g in self.groups])


# ------------------------------------------------------------------------------------------------ hook result
_RESULT_KEYS = ("cache_len_after", "selector_status", "effective_tokens_before", "budget_total",
                "recent_unabsorbed_tokens")


@dataclass(frozen=True)
class PlacementPlan:
    """A successful compaction; ``to_hook_result_dict`` is what ``triattention_apply_compression`` returns."""

    cache_len_after: int
    selector_status: str
    selection_mode: str
    effective_tokens_before: int
    budget_total: int
    recent_unabsorbed_tokens: Optional[int]
    block_reclaim: Optional[ReclaimEvent] = None

    @property
    def reclaimed_block_count(self) -> int:
        return self.block_reclaim.reclaimed_block_count() if self.block_reclaim is not None else 0

    def to_hook_result_dict(self) -> dict:
        out = {"applied": True, "reason": "kv_compacted:" + self.selection_mode}
        out.update((k, getattr(self, k)) for k in _RESULT_KEYS)
        out["block_reclaim"] = self.block_reclaim.to_dict() if self.block_reclaim is not None else None
        out["reclaimed_block_count"] = self.reclaimed_block_count
        return out


# ------------------------------------------------------------------------------------------------ keep selection
def _columns_of_rows(indices: Any) -> int:
    """k of a per-head selection: second extent of a 2-D array, or the length of the first row of a list of lists."""
    if hasattr(indices, "ndim") and hasattr(indices, "shape"):
        if int(indices.ndim) != 2:
            raise ValueError(f"per_head indices tensor must be 2D, got ndim={indices.ndim}")
        return int(indices.shape[1])
    if isinstance(indices, list):
        return len(indices[0]) if indices and isinstance(indices[0], list) else 0
    raise ValueError(f"unsupported per_head indices type: {type(indices).__name__}")


def _flat_count(indices: Any) -> int:
    if hasattr(indices, "numel"):
        return int(indices.numel())
    if isinstance(indices, list):
        return len(indices)
    raise ValueError(f"unsupported shared indices type: {type(indices).__name__}")


@dataclass(frozen=True)
class KeepPlan:
    """A selector's answer: ``mode`` "per_head" (indices ``[Hkv, k]``) or "shared" (``[k]``), and which selection
    semantics produced it."""

    mode: str
    indices: Any
    semantic: Optional[str] = None

    @classmethod
    def from_selector_result(cls, result: dict) -> "KeepPlan":
        semantic = result.get("semantic")
        return cls(str(result.get("mode", "shared")), result.get("indices"), semantic if semantic is None else str(semantic))

    @property
    def selection_mode_label(self) -> str:
        return self.mode + (":" + self.semantic if self.semantic else "")

    def keep_count(self) -> int:
        return _columns_of_rows(self.indices) if self.mode == "per_head" else _flat_count(self.indices)

    def to_selector_result(self) -> dict:
        out = dict(mode=self.mode, indices=self.indices)
        if self.semantic is not None:
            out["semantic"] = self.semantic
        return out
