"""Plan/result records of the hook pipeline; dict layouts match the reference's runtime/plan_models.py:13-134."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional


@dataclass(frozen=True)
class KeepPlan:
    """Keep selection produced by a selector: mode 'per_head' ([Hkv, k]) or 'shared' ([k])."""

    mode: str
    indices: Any
    semantic: Optional[str] = None

    @classmethod
    def from_selector_result(cls, result: dict) -> "KeepPlan":
        sem = result.get("semantic")
        return cls(mode=str(result.get("mode", "shared")), indices=result.get("indices"),
                   semantic=None if sem is None else str(sem))

    @property
    def selection_mode_label(self) -> str:
        return f"{self.mode}:{self.semantic}" if self.semantic else self.mode

    def keep_count(self) -> int:
        idx = self.indices
        if self.mode == "per_head":
            if hasattr(idx, "ndim") and hasattr(idx, "shape"):
                if int(idx.ndim) != 2:
                    raise ValueError(f"per_head indices tensor must be 2D, got ndim={idx.ndim}")
                return int(idx.shape[1])
            if isinstance(idx, list):
                if not idx:
                    return 0
                return len(idx[0]) if isinstance(idx[0], list) else 0
            raise ValueError(f"unsupported per_head indices type: {type(idx).__name__}")
        if hasattr(idx, "numel"):
            return int(idx.numel())
        if isinstance(idx, list):
            return len(idx)
        raise ValueError(f"unsupported shared indices type: {type(idx).__name__}")

    def to_selector_result(self) -> dict:
        out = {"mode": self.mode, "indices": self.indices}
        if self.semantic is not None:
            out["semantic"] = self.semantic
        return out


@dataclass(frozen=True)
class ReclaimGroup:
    gid: int
    block_ids_before: list
    block_ids_after: list
    block_ids_removed: list

    def to_dict(self) -> dict:
        return {"gid": self.gid, "block_ids_before": list(self.block_ids_before),
                "block_ids_after": list(self.block_ids_after), "block_ids_removed": list(self.block_ids_removed)}


@dataclass(frozen=True)
class ReclaimEvent:
    mode: str
    groups: list

    def reclaimed_block_count(self) -> int:
        return sum(len(g.block_ids_removed) for g in self.groups)

    def to_dict(self) -> dict:
        return {"mode": self.mode, "groups": [g.to_dict() for g in self.groups]}


@dataclass(frozen=True)
class PlacementPlan:
    """Result of a successful compaction, rendered as the hook's result dict."""

    cache_len_after: int
    selector_status: str
    selection_mode: str
    effective_tokens_before: int
    budget_total: int
    recent_unabsorbed_tokens: Optional[int]
    block_reclaim: Optional[ReclaimEvent] = None

    @property
    def reclaimed_block_count(self) -> int:
        return 0 if self.block_reclaim is None else self.block_reclaim.reclaimed_block_count()

    def to_hook_result_dict(self) -> dict:
        return {
            "applied": True,
            "reason": f"kv_compacted:{self.selection_mode}",
            "cache_len_after": self.cache_len_after,
            "selector_status": self.selector_status,
            "block_reclaim": None if self.block_reclaim is None else self.block_reclaim.to_dict(),
            "effective_tokens_before": self.effective_tokens_before,
            "budget_total": self.budget_total,
            "reclaimed_block_count": self.reclaimed_block_count,
            "recent_unabsorbed_tokens": self.recent_unabsorbed_tokens,
        }
