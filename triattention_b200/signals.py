"""Signal exchanged between scheduler and model runner (same fields as the reference's runtime/signals.py:12-26)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

TriggerReason = Literal["none", "length_threshold", "kv_usage_threshold"]


@dataclass(frozen=True)
class CompressionSignal:
    """Per-request compression signal for one scheduler step."""

    req_id: str
    should_compress: bool
    reason: TriggerReason
    estimated_cache_len: int
    step: int
    kv_usage: Optional[float]
    protect_prefill: bool
    prefill_len: int
    scheduled_tokens: int = 1
