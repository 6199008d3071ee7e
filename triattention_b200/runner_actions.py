"""Worker-side driver of a step's compression actions.

Mirror of the reference's ``runtime/runner_compression_actions.py:11-237`` (``execute_runner_compression_actions``)
and ``runtime/executor.py:11-84`` with one difference: where the reference executes the triggered requests one
after the other, this driver hands all of them to the runner's batched hook
(``triattention_apply_compression_batch``, installed by ``hook.install_runner_compression_hook``) so that the
native work of a step is ONE call.  Everything the scheduler and the state store see is unchanged: the
batch-queue de-duplication rule, the strict-mode errors, the ``mark_compressed`` / ``mark_compression_skipped``
bookkeeping and the event dictionaries (keys and values) are those of the reference, in the order of ``signals``.
"""
from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from typing import Any, Optional

from .constants import TRITON_SCORING_REQUIRED_MARKER
from .signals import CompressionSignal


@dataclass(frozen=True)
class CompressionExecutionResult:
    """What an executor reports for one request (runtime/executor.py:11-16)."""
    applied: bool
    reason: str
    cache_len_after: Optional[int] = None
    details: Optional[dict] = None


def _result_from_hook(value: Any) -> CompressionExecutionResult:
    # the hook may answer with a bool or with its result dictionary (runtime/executor.py:55-84)
    if isinstance(value, bool):
        return CompressionExecutionResult(applied=value, reason="applied" if value else "runner_hook_rejected")
    if isinstance(value, dict):
        details = dict(value)
        return CompressionExecutionResult(
            applied=bool(details.get("applied", False)), reason=str(details.get("reason", "runner_hook_result")),
            cache_len_after=details.get("cache_len_after"), details=details)
    return CompressionExecutionResult(applied=False, reason=f"unsupported_hook_result:{type(value).__name__}")


class RunnerHookCompressionExecutor:
    """Executor over the runner's hooks: ``execute`` is the reference's per-request contract, ``execute_batch``
    runs all requests of a step through the batched hook when the runner has one."""

    hook_name = "triattention_apply_compression"
    batch_hook_name = "triattention_apply_compression_batch"

    def __init__(self, base_runner: Any):
        self._base_runner = base_runner

    def execute(self, req_id, signal: CompressionSignal, scheduler_output: Any) -> CompressionExecutionResult:
        hook = getattr(self._base_runner, self.hook_name, None)
        if not callable(hook):
            return CompressionExecutionResult(applied=False, reason="runner_hook_missing")
        return _result_from_hook(hook(req_id=req_id, signal=signal, scheduler_output=scheduler_output))

    def execute_batch(self, requests: list, scheduler_output: Any) -> dict:
        """{req_id: CompressionExecutionResult} for ``requests`` = [(req_id, signal), ...]."""
        batch = getattr(self._base_runner, self.batch_hook_name, None)
        if callable(batch):
            out = batch(requests, scheduler_output)
            return {req_id: _result_from_hook(out.get(req_id)) for req_id, _ in requests}
        return {req_id: self.execute(req_id, signal, scheduler_output) for req_id, signal in requests}


def _event(req_id, signal, status: str, reason: str, cache_len_after, **more) -> dict:
    ev = {"req_id": req_id, "step": signal.step, "status": status, "reason": reason, "cache_len_after": cache_len_after}
    ev.update(more)
    ev.update(scheduled_tokens=int(getattr(signal, "scheduled_tokens", 1)),
              estimated_cache_len=int(getattr(signal, "estimated_cache_len", 0)),
              prefill_len=int(getattr(signal, "prefill_len", 0)))
    return ev


def _scheduler_num_computed(scheduler_output: Any, req_id) -> Optional[int]:
    cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
    ids, nct = getattr(cached, "req_ids", None), getattr(cached, "num_computed_tokens", None)
    if isinstance(ids, list) and isinstance(nct, list):
        try:
            return int(nct[ids.index(req_id)])
        except (ValueError, IndexError):
            return None
    return None


def _is_duplicate_trigger(req_state: Any, signal: CompressionSignal) -> bool:
    """Batch-queue race guard (runner_compression_actions.py:26-41): a second signal for a request that was
    compressed in the previous step, outside chunked prefill, must not run again."""
    if req_state is None:
        return False
    last_step = getattr(req_state, "last_compression_step", -1)
    count = int(getattr(req_state, "compression_count", 0) or 0)
    return (count > 0 and last_step >= 0 and signal.step - last_step <= 1
            and int(getattr(signal, "scheduled_tokens", 1)) <= 1)


def execute_runner_compression_actions(*, executor: Any, state_store: Any, scheduler_output: Any,
                                       signals: dict, strict_no_downgrade: bool, allowed_strict_skip_reasons: set,
                                       logger: logging.Logger, log_decisions: bool) -> list:
    """Run the compression of every triggered request of a step and return the scheduler-side events."""
    events: list = []
    todo, duplicates = [], {}
    for req_id, signal in signals.items():
        if not signal.should_compress:
            continue
        req_state = state_store.get(req_id) if hasattr(state_store, "get") else None
        if _is_duplicate_trigger(req_state, signal):
            duplicates[req_id] = req_state
        else:
            todo.append((req_id, signal))

    results: dict = {}
    errors: dict = {}
    run_batch = getattr(executor, "execute_batch", None)
    if callable(run_batch) and len(todo) > 1:
        try:
            results = run_batch(todo, scheduler_output)
        except Exception as exc:  # the whole native step failed: every request of the batch reports it
            errors = {req_id: exc for req_id, _ in todo}
    else:
        for req_id, signal in todo:
            try:
                results[req_id] = executor.execute(req_id=req_id, signal=signal, scheduler_output=scheduler_output)
            except Exception as exc:
                errors[req_id] = exc

    # bookkeeping and events in the order of `signals`, as the reference's loop produces them
    for req_id, signal in signals.items():
        if not signal.should_compress:
            continue
        if req_id in duplicates:
            req_state = duplicates[req_id]
            logger.info("TriAttention compression skipped (batch-queue dedup) req=%s step=%d last_compression_step=%d",
                        req_id, signal.step, getattr(req_state, "last_compression_step", -1))
            if hasattr(state_store, "mark_compression_skipped"):
                state_store.mark_compression_skipped(req_id=req_id, reason="batch_queue_dedup", step=signal.step)
            events.append(_event(req_id, signal, "skipped", "batch_queue_dedup",
                                 getattr(req_state, "current_cache_len", None)))
            continue
        exc = errors.get(req_id)
        if exc is not None:
            if strict_no_downgrade:
                logger.error("TriAttention strict mode fatal: compression executor exception req=%s step=%d",
                             req_id, signal.step, exc_info=exc)
                raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:executor_exception:req={req_id}:"
                                   f"step={signal.step}:type={type(exc).__name__}") from exc
            if TRITON_SCORING_REQUIRED_MARKER in str(exc):
                logger.error("TriAttention fatal: Triton scoring is required. req=%s step=%d", req_id, signal.step,
                             exc_info=exc)
                raise exc
            reason = f"executor_exception:{type(exc).__name__}"
            state_store.mark_compression_skipped(req_id=req_id, reason=reason, step=signal.step)
            logger.error("TriAttention compression executor failed req=%s step=%d", req_id, signal.step, exc_info=exc)
            events.append(_event(req_id, signal, "error", reason, None))
            continue

        result = results[req_id]
        if strict_no_downgrade and not result.applied and result.reason not in allowed_strict_skip_reasons:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:unexpected_skip:req={req_id}:step={signal.step}:"
                               f"reason={result.reason}")
        details = result.details if isinstance(result.details, dict) else {}
        reclaim = result.details.get("block_reclaim") if isinstance(result.details, dict) else None
        if result.applied:
            cache_len_after = signal.estimated_cache_len if result.cache_len_after is None else result.cache_len_after
            before_len = details.get("effective_tokens_before")
            logger.info("TriAttention compression applied req=%s step=%d reason=%s before=%s after=%d reclaimed_blocks=%s",
                        req_id, signal.step, result.reason, before_len, cache_len_after,
                        details.get("reclaimed_block_count"))
            state_store.mark_compressed(req_id=req_id, step=signal.step, cache_len=cache_len_after,
                                        scheduled_tokens=int(getattr(signal, "scheduled_tokens", 1)),
                                        scheduler_nct=_scheduler_num_computed(scheduler_output, req_id))
            if log_decisions:
                logger.debug("TriAttention compression summary req=%s step=%d before=%s after=%d budget=%s "
                             "reclaimed_blocks=%s recent_unabsorbed=%s scheduled_tokens=%s estimated_cache_len=%s reason=%s",
                             req_id, signal.step, before_len, cache_len_after, details.get("budget_total"),
                             details.get("reclaimed_block_count"), details.get("recent_unabsorbed_tokens"),
                             int(getattr(signal, "scheduled_tokens", 1)), int(getattr(signal, "estimated_cache_len", 0)),
                             result.reason)
            events.append(_event(req_id, signal, "applied", result.reason, cache_len_after,
                                 details=result.details, block_reclaim=reclaim))
        else:
            state_store.mark_compression_skipped(req_id=req_id, reason=result.reason, step=signal.step)
            logger.info("TriAttention compression skipped req=%s step=%d reason=%s cache_len_after=%s details=%s",
                        req_id, signal.step, result.reason, result.cache_len_after, result.details)
            events.append(_event(req_id, signal, "skipped", result.reason, result.cache_len_after,
                                 details=result.details, block_reclaim=reclaim))
    return events


# ------------------------------------------------------------------------------------------ step life cycle
# What the worker does with a scheduler output BEFORE the actions of the step: keep the request-state store in step
# with arrivals, departures, preemptions and with the cache lengths the signals report (the reference's
# runtime/runner_state_updates.py:20-128).  The hook reads the lengths kept here.
# read once at import, like the reference's module constant (runner_state_updates.py:10-13)
LEGACY_COMPRESSED_ESTIMATE = os.environ.get("TRIATTN_RUNTIME_LEGACY_COMPRESSED_ESTIMATE", "0").strip().lower() in {
    "1", "true", "yes", "on"}


def full_prefill_len(request_like: Any) -> int:
    """Prompt length of a new request from whichever field the engine version carries; the largest wins."""
    seen = [0]
    for attr in ("prompt_token_ids", "prefill_token_ids"):
        ids = getattr(request_like, attr, None)
        if ids is not None:
            try:
                seen.append(len(ids))
            except Exception:
                pass
    for attr in ("prompt_token_ids_len", "num_prompt_tokens"):
        raw = getattr(request_like, attr, None)
        if raw is not None:
            try:
                seen.append(int(raw))
            except (TypeError, ValueError):
                pass
    return max(seen)


def register_new_requests(*, state_store: Any, scheduler_output: Any, protect_prefill: bool) -> None:
    for new_req in scheduler_output.scheduled_new_reqs:
        state_store.ensure(req_id=new_req.req_id, prefill_len=full_prefill_len(new_req), protect_prefill=protect_prefill)


def cleanup_finished_requests(*, state_store: Any, scheduler_output: Any) -> None:
    for req_id in scheduler_output.finished_req_ids:
        state_store.remove(req_id)


def mark_preemptions(*, state_store: Any, scheduler_output: Any) -> None:
    for req_id in getattr(scheduler_output, "preempted_req_ids", None) or ():
        state_store.mark_preempted(req_id)


def mark_resumed(*, state_store: Any, scheduler_output: Any) -> None:
    cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
    if cached is None:
        return
    resumed = getattr(cached, "resumed_req_ids", None)
    if resumed is None:
        resumed = getattr(cached, "req_ids", []) or []
    for req_id in resumed:
        state_store.mark_resumed(req_id)


def consume_runner_signals(*, state_store: Any, scheduler_output: Any, last_step: int, logger: logging.Logger,
                           log_decisions: bool, legacy_compressed_estimate: Optional[bool] = None) -> tuple:
    """``(step, signals)`` of the scheduler output, after recording every signal in the store.

    Before a request's first compression its cache length is the scheduler's estimate; afterwards the worker keeps its
    own count (previous length + tokens scheduled in this step), because the scheduler's snapshots may lag the
    compaction in asynchronous scheduling.  ``legacy_compressed_estimate`` restores the scheduler's estimate; left at
    None it follows the environment switch TRIATTN_RUNTIME_LEGACY_COMPRESSED_ESTIMATE, as the reference does."""
    if legacy_compressed_estimate is None:
        legacy_compressed_estimate = LEGACY_COMPRESSED_ESTIMATE
    step = getattr(scheduler_output, "triattention_step", last_step + 1)
    signals = getattr(scheduler_output, "triattention_signals", {})
    for req_id, signal in signals.items():
        state = state_store.ensure(req_id=req_id, prefill_len=signal.prefill_len, protect_prefill=signal.protect_prefill)
        estimate = max(0, int(signal.estimated_cache_len))
        if int(getattr(state, "compression_count", 0)) > 0 and not legacy_compressed_estimate:
            estimate = max(0, int(getattr(state, "current_cache_len", 0))) + max(0, int(getattr(signal, "scheduled_tokens", 1)))
        state_store.update_cache_len(req_id, estimate, step=signal.step)
        if signal.should_compress:
            state_store.mark_trigger(req_id, signal.reason, signal.step)
            if log_decisions:
                logger.debug("TriAttention trigger req=%s step=%d reason=%s len=%d mode=%s", req_id, signal.step,
                             signal.reason, signal.estimated_cache_len, state.mode)
    return step, signals
