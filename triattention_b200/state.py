"""Per-request bookkeeping of the compression runtime.

Same fields and transitions as the reference's ``runtime/state.py:9-153`` (``RequestCompressionState``,
``RequestStateStore``): the hook reads ``compression_count``, ``current_cache_len`` and ``last_absorbed_cache_len``
from these records (hook_runtime_context.py:139-176), the worker-side driver reads ``last_compression_step`` for its
de-duplication rule and writes them through ``mark_compressed`` / ``mark_compression_skipped``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, Optional


@dataclass
class RequestCompressionState:
    req_id: str
    prefill_len: int
    protect_prefill: bool
    current_cache_len: int = 0
    last_absorbed_cache_len: int = 0          # cache length right after the last compression (prefill before the first)
    recent_unabsorbed_tokens: int = 0         # tokens appended since
    compression_count: int = 0
    last_compression_step: int = -1
    pending_triggers: int = 0
    last_trigger_reason: str = "none"
    is_preempted: bool = False
    current_cache_len_semantics: str = "unknown"
    current_cache_len_step: int = -1
    nct_at_last_compression: Optional[int] = None           # scheduler's num_computed_tokens at that moment
    cache_len_after_last_compression: Optional[int] = None

    @property
    def mode(self) -> str:
        return "protect_prefill" if self.protect_prefill else "trim_prefill"


class RequestStateStore:
    """Records keyed by request id; every mutator is a no-op for an unknown request."""

    def __init__(self) -> None:
        self._states: Dict[str, RequestCompressionState] = {}
        self._compressed_req_ids: set = set()

    def _update(self, req_id: str, change: Callable[[RequestCompressionState], None]) -> None:
        state = self._states.get(req_id)
        if state is not None:
            change(state)

    # ---- life cycle
    def ensure(self, req_id: str, prefill_len: int, protect_prefill: bool) -> RequestCompressionState:
        state = self._states.get(req_id)
        if state is None:
            state = self._states[req_id] = RequestCompressionState(
                req_id=req_id, prefill_len=prefill_len, protect_prefill=protect_prefill,
                last_absorbed_cache_len=max(0, prefill_len))
            return state
        # keep the largest prefill length seen and the latest mode; until the first compression the prefill is
        # the absorbed baseline
        state.prefill_len = max(state.prefill_len, prefill_len)
        state.protect_prefill = protect_prefill
        if state.compression_count <= 0:
            state.last_absorbed_cache_len = max(state.last_absorbed_cache_len, state.prefill_len)
        return state

    def remove(self, req_id: str) -> None:
        self._states.pop(req_id, None)
        self._compressed_req_ids.discard(req_id)

    def mark_preempted(self, req_id: str) -> None:
        self._update(req_id, lambda s: setattr(s, "is_preempted", True))

    def mark_resumed(self, req_id: str) -> None:
        self._update(req_id, lambda s: setattr(s, "is_preempted", False))

    # ---- per step
    def update_cache_len(self, req_id: str, cache_len: int, step: Optional[int] = None) -> None:
        def change(s: RequestCompressionState) -> None:
            s.current_cache_len = max(0, int(cache_len))
            s.current_cache_len_semantics = "estimated_with_scheduled"
            if isinstance(step, int):
                s.current_cache_len_step = step
            s.recent_unabsorbed_tokens = max(0, s.current_cache_len - max(0, int(s.last_absorbed_cache_len)))
        self._update(req_id, change)

    def mark_trigger(self, req_id: str, reason: str, step: int) -> None:
        # the step is NOT recorded here: this runs before the actions of the step, and the de-duplication rule
        # compares the step of the last APPLIED compression
        def change(s: RequestCompressionState) -> None:
            s.pending_triggers += 1
            s.last_trigger_reason = reason
        self._update(req_id, change)

    def mark_compressed(self, req_id: str, step: int, cache_len: int, scheduled_tokens: int = 0,
                        scheduler_nct: Optional[int] = None) -> None:
        def change(s: RequestCompressionState) -> None:
            self._compressed_req_ids.add(req_id)
            s.compression_count += 1
            s.pending_triggers = max(s.pending_triggers - 1, 0)
            s.last_compression_step = step
            # the tokens decoded in the compression step itself are already in the cache when the next step starts
            s.current_cache_len = cache_len + max(0, scheduled_tokens)
            s.current_cache_len_semantics = "estimated_with_scheduled"
            s.current_cache_len_step = int(step)
            s.last_absorbed_cache_len = max(0, int(cache_len))
            s.recent_unabsorbed_tokens = 0
            s.last_trigger_reason = "applied"
            s.cache_len_after_last_compression = int(cache_len)
            if scheduler_nct is not None:
                s.nct_at_last_compression = int(scheduler_nct)
        self._update(req_id, change)

    def mark_compression_skipped(self, req_id: str, reason: str, step: int) -> None:
        def change(s: RequestCompressionState) -> None:
            s.pending_triggers = max(s.pending_triggers - 1, 0)
            s.last_trigger_reason = f"skipped:{reason}"
        self._update(req_id, change)

    # ---- queries
    def get(self, req_id: str) -> Optional[RequestCompressionState]:
        return self._states.get(req_id)

    def snapshot(self) -> Dict[str, RequestCompressionState]:
        return dict(self._states)

    def has_active_compressed_requests(self) -> bool:
        return bool(self._compressed_req_ids)

    def has_compressed_request_in(self, req_ids: Iterable[str]) -> bool:
        return any(r in self._compressed_req_ids for r in req_ids)
