"""Effective cache lengths for the forward pass after a compaction.

A compressed request holds fewer tokens in its cache than the engine's ``num_computed_tokens`` says, so the
sequence length and the slot-mapping positions of its next forward pass must be computed from the *effective*
length.  This module derives, from the request-state store and the scheduler output of the step, the sparse
overrides that ``input_patch_ops`` applies on the device: rules and return convention of the reference's
``runtime/effective_overrides.py:209-359`` (``build_effective_sparse_overrides``), with the request-key
normalisation of ``runtime/request_key_compat.py:16-69`` and the row lookup of
``runtime/runner_struct_compat.py:20-55``.
"""
from __future__ import annotations

from typing import Any, Optional

_ITEMS_ATTR = "_triattention_cached_scheduled_token_items"
_RESULT_ATTR = "_triattention_cached_sparse_overrides"
NO_OVERRIDES = (None, None, None, 0)


def _req_id_of(key: Any):
    if isinstance(key, (str, int)):
        return key
    for attr in ("request_id", "req_id"):
        value = getattr(key, attr, None)
        if isinstance(value, (str, int)):
            return value
    return None


def scheduled_token_items(scheduler_output: Any) -> list:
    """``[(raw key, req_id, scheduled tokens)]`` in the scheduler's order; remembered on the output object."""
    if scheduler_output is None:
        return []
    try:
        cached = getattr(scheduler_output, _ITEMS_ATTR, None)
    except Exception:
        cached = None
    if isinstance(cached, list):
        return cached
    items = []
    scheduled = getattr(scheduler_output, "num_scheduled_tokens", None)
    if isinstance(scheduled, dict):
        for key, value in scheduled.items():
            req_id = _req_id_of(key)
            if req_id is None:
                continue
            try:
                items.append((key, req_id, int(value)))
            except (TypeError, ValueError):
                continue
    try:
        setattr(scheduler_output, _ITEMS_ATTR, items)
    except Exception:
        pass
    return items


def req_id_to_index(base_runner: Any) -> Optional[dict]:
    """Request id -> row of the runner's batch arrays: ``req_states``, else ``input_batch``, else its id list."""
    input_batch = getattr(base_runner, "input_batch", None)
    for holder in (getattr(base_runner, "req_states", None), input_batch):
        table = getattr(holder, "req_id_to_index", None) if holder is not None else None
        if isinstance(table, dict) and table:
            return table
    if input_batch is None:
        return None
    ids = getattr(input_batch, "req_ids", None)
    try:
        ids = ids() if callable(ids) else ids
    except Exception:
        ids = None
    if not isinstance(ids, list):
        ids = getattr(input_batch, "_req_ids", None)
    if not isinstance(ids, list):
        return None
    return {r: i for i, r in enumerate(ids) if r is not None} or None


def _pre_step_marker(state: Any, scheduler_step: Optional[int]) -> Optional[bool]:
    """Does ``current_cache_len`` already exclude this step's tokens?  None when the record carries no marker."""
    semantics = getattr(state, "current_cache_len_semantics", None) if state is not None else None
    if not isinstance(semantics, str):
        return None
    if semantics != "effective_pre_step":
        return False
    state_step = getattr(state, "current_cache_len_step", None)
    if isinstance(scheduler_step, int) and isinstance(state_step, int):
        return state_step == scheduler_step
    return True


def effective_base_before_step(state: Any, abs_progress: int, scheduled_tokens: int,
                               scheduler_step: Optional[int]) -> int:
    """Tokens in the cache before this step's tokens are appended (effective_overrides.py:73-96)."""
    current = int(getattr(state, "current_cache_len", abs_progress)) if state is not None else abs_progress
    marked = _pre_step_marker(state, scheduler_step)
    if marked is True:
        return current
    if marked is None and state is not None:
        count = getattr(state, "compression_count", None)
        if isinstance(count, int) and count > 0:
            raise RuntimeError("TRIATTN_EFFECTIVE_BASE_STATE_SEMANTICS_MISSING:"
                               "compressed_request_state_missing_current_cache_len_semantics")
    return max(0, current - max(0, int(scheduled_tokens)))


def _abs_progress(req_state: Any, state: Any, scheduled_tokens: int, scheduler_step: Optional[int],
                  scheduler_nct: Optional[int]) -> int:
    """The engine's own progress counter for the request (effective_overrides.py:120-162): the scheduler's value
    for this step when it is known, else the runner's; a compressed request whose counter still lags its prompt
    by one prefill chunk on its first decode step is clamped to the prompt length."""
    if scheduler_nct is not None:
        progress = int(scheduler_nct)
    else:
        progress = int(getattr(req_state, "num_computed_tokens", 0)) if req_state is not None else 0
    if state is None:
        return progress
    count, prefill_len = getattr(state, "compression_count", None), getattr(state, "prefill_len", None)
    if not isinstance(count, int) or count <= 0 or not isinstance(prefill_len, int) or prefill_len <= 0:
        return progress
    if progress >= prefill_len:
        return progress
    if int(scheduled_tokens) == 1 and _pre_step_marker(state, scheduler_step) is True:
        return int(prefill_len)
    return progress


def _remember(scheduler_output: Any, key, value):
    if scheduler_output is not None:
        try:
            cache = getattr(scheduler_output, _RESULT_ATTR, None)
            if not isinstance(cache, dict):
                cache = {}
                setattr(scheduler_output, _RESULT_ATTR, cache)
            cache[key] = value
        except Exception:
            pass
    return value


def build_effective_sparse_overrides(*, base_runner: Any, state_store: Any, scheduler_output: Any,
                                     compression_events: Optional[list] = None) -> tuple:
    """``(seq_bases, pos_deltas, single_seq_base, single_pos_delta)`` for the step.

    ``seq_bases[row]`` = effective cache length of the request in that row before the step, ``pos_deltas[row]`` =
    that length minus the engine's absolute progress; only rows with a non-zero delta are listed, ``None`` stands
    for an empty dict, and the last two values repeat the single entry when there is exactly one.  The result is
    remembered on ``scheduler_output`` for the (runner, store) pair.
    """
    key = (id(base_runner), id(state_store))
    if scheduler_output is not None:
        try:
            cache = getattr(scheduler_output, _RESULT_ATTR, None)
        except Exception:
            cache = None
        hit = cache.get(key) if isinstance(cache, dict) else None
        if isinstance(hit, tuple) and len(hit) == 4:
            return hit
    requests = getattr(base_runner, "requests", None)
    if not isinstance(requests, dict):
        return _remember(scheduler_output, key, NO_OVERRIDES)
    rows = req_id_to_index(base_runner)
    if not isinstance(rows, dict):
        return _remember(scheduler_output, key, NO_OVERRIDES)

    any_compressed = None
    checker = getattr(state_store, "has_active_compressed_requests", None) if state_store is not None else None
    if callable(checker):
        try:
            any_compressed = bool(checker())
        except Exception:
            any_compressed = None
    applied = {e["req_id"] for e in compression_events or []
               if isinstance(e, dict) and e.get("status") == "applied" and e.get("req_id") is not None} \
        if isinstance(compression_events, list) else set()
    if any_compressed is False and applied:
        raise RuntimeError("TRIATTN_COMPRESSION_EVENT_STATE_MISMATCH:"
                           "applied_compression_events_present_but_state_store_reports_no_compressed_requests")
    if any_compressed is False:
        return _remember(scheduler_output, key, NO_OVERRIDES)
    items = scheduled_token_items(scheduler_output)
    if not items:
        return _remember(scheduler_output, key, NO_OVERRIDES)

    step = getattr(scheduler_output, "triattention_step", None)
    step = int(step) if isinstance(step, int) else None
    nct_map = None
    cached_reqs = getattr(scheduler_output, "scheduled_cached_reqs", None)
    if cached_reqs is not None:
        ids, ncts = getattr(cached_reqs, "req_ids", None), getattr(cached_reqs, "num_computed_tokens", None)
        if isinstance(ids, list) and isinstance(ncts, list) and len(ids) == len(ncts):
            nct_map = dict(zip(ids, ncts))
    get_state = getattr(state_store, "get", None)
    get_state = get_state if callable(get_state) else None

    seq_bases, pos_deltas = {}, {}
    for _raw, req_id, scheduled in items:
        row = rows.get(req_id)
        if not isinstance(row, int):
            continue
        state = get_state(req_id) if get_state is not None else None
        if state is not None:
            count = getattr(state, "compression_count", None)
            if isinstance(count, int) and count <= 0:
                continue  # never compressed: the engine's own lengths hold
        nct_then = getattr(state, "nct_at_last_compression", None) if state is not None else None
        len_then = getattr(state, "cache_len_after_last_compression", None) if state is not None else None
        nct_now = nct_map.get(req_id) if nct_map is not None else None
        if isinstance(nct_then, int) and isinstance(len_then, int) and isinstance(nct_now, int):
            # anchored at the last compression: the delta stays constant until the next one
            base = len_then + (nct_now - nct_then)
            delta = int(len_then - nct_then)
        else:
            progress = _abs_progress(requests.get(req_id), state, scheduled, step, nct_now)
            base = effective_base_before_step(state, progress, scheduled, step)
            delta = int(base - progress)
        if delta != 0:
            seq_bases[row] = base
            pos_deltas[row] = delta

    single_base, single_delta = None, 0
    if len(seq_bases) == 1:
        single_base = next(iter(seq_bases.values()))
        single_delta = int(next(iter(pos_deltas.values())))
    return _remember(scheduler_output, key, (seq_bases or None, pos_deltas or None, single_base, single_delta))
