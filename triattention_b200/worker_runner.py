"""The worker's model-runner proxy: one ``execute_model`` call of the serving engine, with the compression step in it.

Order of a step (the reference's ``runtime/runner.py:358-410``): request-state bookkeeping -> signals of the
scheduler -> self-triggers the scheduler missed -> compression actions (ALL triggered requests in one native call
through the batched hook) -> worker block tables shrunk -> stale ``new_block_ids`` trimmed -> the engine's own
``execute_model`` under the effective-length overrides -> events attached to the output for the scheduler.

The pieces are plain functions over the attributes the reference reads, and :class:`TriAttentionModelRunner` strings
them together with the reference's constructor and method names.  The one engine-specific seam - how the patched
input preparation of the engine learns the overrides of the step - is a context manager that can be replaced
(``override_scope``); the default publishes them through :func:`current_effective_input_overrides`.
"""
from __future__ import annotations

import logging
import os
import time
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Callable, Iterator, Optional

from . import effective_overrides as _eo
from . import runner_actions as _ra
from .config import TriAttentionRuntimeConfig
from .perf_profile import TriAttentionPerfProfile
from .signals import CompressionSignal
from .state import RequestStateStore
from .worker_reclaim_sync import apply_worker_block_reclaim_events

EVENTS_ATTR = "triattention_compression_events"
STRICT_SKIP_REASONS = frozenset({"under_budget", "prefill_exceeds_budget", "req_state_not_found", "batch_queue_dedup"})

_log = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------------ block-table views
def _first_block_table(base_runner: Any):
    """``(input_batch, block-table object, its first inner table)`` of the runner, None where missing."""
    batch = getattr(base_runner, "input_batch", None)
    table = getattr(batch, "block_table", None) if batch is not None else None
    if table is None:
        return batch, None, None
    inner = getattr(table, "block_tables", None)
    return batch, table, (inner[0] if isinstance(inner, list) and inner else table)


def actual_kv_from_block_table(base_runner: Any, req_id: Any) -> Optional[int]:
    """Tokens the request's blocks can hold on THIS worker (blocks in its row x block size): free of the lag the
    scheduler's counters have under asynchronous scheduling.  None when the row cannot be found
    (``runtime/runner.py:92-124``)."""
    batch, _table, first = _first_block_table(base_runner)
    rows = getattr(batch, "req_id_to_index", None) if batch is not None else None
    if not isinstance(rows, dict):
        return None
    row = rows.get(req_id)
    if not isinstance(row, int) or first is None:
        return None
    counts = getattr(first, "num_blocks_per_row", None)
    if counts is None:
        return None
    block_size = int(getattr(getattr(base_runner, "cache_config", None), "block_size", 0))
    return int(counts[row]) * block_size if block_size > 0 else None


# ------------------------------------------------------------------------------------------------ self-triggers
def supplement_worker_self_triggers(*, base_runner: Any, config: Any, state_store: Any, scheduler_output: Any,
                                    signals: dict, last_step: int, logger: logging.Logger = _log) -> dict:
    """Add (or correct) triggers from what the worker itself knows (``runtime/runner.py:126-210``).

    A decode-step trigger of the scheduler stands.  Otherwise the request's length is, in this order: the worker's
    own count once it has been compressed; the capacity of its block-table row (which already covers the tokens of
    this step); the runner's ``num_computed_tokens`` plus the tokens of this step.  At or above the scheduler's
    threshold the request gets a ``length_threshold`` signal with that length.
    """
    if not config.enable_experimental_kv_compaction:
        return signals
    get_state = getattr(state_store, "get", None)
    for _key, req_id, scheduled in _eo.scheduled_token_items(scheduler_output):
        have = signals.get(req_id)
        if have is not None and have.should_compress and int(getattr(have, "scheduled_tokens", 1)) <= 1:
            continue
        state = get_state(req_id) if get_state is not None else None
        if state is None:
            continue
        step_tokens = max(1, int(scheduled))
        from_blocks = False
        if state.compression_count > 0 and state.current_cache_len > 0:
            length = state.current_cache_len
        else:
            length = actual_kv_from_block_table(base_runner, req_id)
            from_blocks = length is not None
            if length is None:
                requests = getattr(base_runner, "requests", None)
                req = requests.get(req_id) if isinstance(requests, dict) else None
                if req is None:
                    continue
                length = int(getattr(req, "num_computed_tokens", 0))
        threshold = config.kv_budget + config.divide_length
        if config.protect_prefill and not config.include_prefill_in_budget:
            threshold += max(state.prefill_len, 0)
        effective = length if from_blocks else length + step_tokens
        if effective < threshold:
            continue
        logger.info("TriAttention worker self-trigger: req=%s actual_kv=%d effective_kv=%d scheduled=%d threshold=%d "
                    "from_blocks=%s", req_id, length, effective, scheduled, threshold, from_blocks)
        signals[req_id] = CompressionSignal(
            req_id=req_id, should_compress=True, reason="length_threshold", estimated_cache_len=effective,
            step=last_step, kv_usage=None, protect_prefill=config.protect_prefill, prefill_len=state.prefill_len,
            scheduled_tokens=step_tokens)
    return signals


# ------------------------------------------------------------------------------------------------ stale new blocks
def trim_new_block_ids_for_compressed_reqs(*, base_runner: Any, state_store: Any, scheduler_output: Any,
                                           logger: logging.Logger = _log) -> None:
    """A scheduler that has not yet seen a reclaim may send a compressed request more new block ids than its
    (shrunk) row can take: cut every group's list to the room that is left (``runtime/runner.py:235-307``)."""
    cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
    req_ids = getattr(cached, "req_ids", None) if cached is not None else None
    new_lists = getattr(cached, "new_block_ids", None) if cached is not None else None
    if not isinstance(req_ids, list) or not isinstance(new_lists, list) or len(req_ids) != len(new_lists):
        return
    batch, table, first = _first_block_table(base_runner)
    if table is None:
        return
    capacity = getattr(table, "max_num_blocks_per_req", None)
    if not isinstance(capacity, int) or capacity <= 0:
        return
    counts = getattr(first, "num_blocks_per_row", None)
    rows = getattr(batch, "req_id_to_index", None)
    if not isinstance(rows, dict):
        return
    for i, req_id in enumerate(req_ids):
        state = state_store.get(req_id)
        if state is None or state.compression_count <= 0 or new_lists[i] is None:
            continue
        row = rows.get(req_id)
        if not isinstance(row, int) or counts is None or not isinstance(new_lists[i], (list, tuple)):
            continue
        held = int(counts[row])
        longest = max(len(g) if isinstance(g, (list, tuple)) else 0 for g in new_lists[i])
        if held + longest <= capacity:
            continue
        room = max(0, capacity - held)
        new_lists[i] = tuple(list(g)[:room] if isinstance(g, (list, tuple)) else g for g in new_lists[i])
        logger.info("TriAttention patched new_block_ids: req=%s current_blocks=%d max=%d new_trimmed=%d->%d", req_id,
                    held, capacity, longest, room)


def needs_effective_input_overrides(state_store: Any, scheduler_output: Any) -> bool:
    """Does this step schedule a request that has been compressed?  (``runtime/runner.py:309-331``)"""
    req_ids = [req_id for _key, req_id, _n in _eo.scheduled_token_items(scheduler_output)]
    if not req_ids:
        return False
    for name, args in (("has_compressed_request_in", (req_ids,)), ("has_active_compressed_requests", ())):
        checker = getattr(state_store, name, None)
        if callable(checker):
            try:
                return bool(checker(*args))
            except Exception:
                return False
    return False


# ------------------------------------------------------------------------------------------------ overrides of a step
@dataclass(frozen=True)
class EffectiveInputOverrides:
    """Sparse overrides of a step plus the rows and query lengths the patched input preparation must meet
    (``runtime/input_adapter.py:24-46``)."""

    seq_base_map: Optional[dict]
    pos_delta_map: Optional[dict]
    single_seq_base: Optional[int]
    single_pos_delta: int
    expected_req_row_indices: Optional[tuple] = None
    expected_query_lens: Optional[tuple] = None

    @property
    def empty(self) -> bool:
        return (self.seq_base_map is None and self.pos_delta_map is None and self.single_seq_base is None
                and self.single_pos_delta == 0)


def prepare_effective_input_overrides(*, base_runner: Any, state_store: Any, scheduler_output: Any) -> EffectiveInputOverrides:
    """``runtime/input_adapter.py:60-108``: the sparse overrides, and - in scheduling order - the batch rows (and
    their scheduled tokens) they apply to; with overrides but no way to find rows the step cannot be patched."""
    rows = _eo.req_id_to_index(base_runner)
    bases, deltas, one_base, one_delta = _eo.build_effective_sparse_overrides(
        base_runner=base_runner, state_store=state_store, scheduler_output=scheduler_output, compression_events=None)
    want_rows = want_lens = None
    if isinstance(rows, dict):
        touched = set(bases or {}) | set(deltas or {})
        picked = [(int(rows[r]), int(n)) for _key, r, n in _eo.scheduled_token_items(scheduler_output)
                  if isinstance(rows.get(r), int) and (not touched or int(rows[r]) in touched)]
        if picked:
            want_rows, want_lens = tuple(p[0] for p in picked), tuple(p[1] for p in picked)
    elif bases or deltas:
        raise RuntimeError("TRIATTN_EXPECTED_REQ_ROW_INDEX_UNAVAILABLE:req_id_to_index_missing_while_overrides_active")
    return EffectiveInputOverrides(bases, deltas, one_base, one_delta, want_rows, want_lens)


_ACTIVE: Optional[EffectiveInputOverrides] = None
_FLAGS = {"consumed": False, "validated": False}  # of the scope in progress: seen by the patched input preparation / checked once


def current_effective_input_overrides() -> Optional[EffectiveInputOverrides]:
    """The overrides of the ``execute_model`` call in progress (None outside one, or when the step has none)."""
    return _ACTIVE


def mark_effective_overrides_consumed() -> None:
    _FLAGS["consumed"] = True


def effective_overrides_consumed() -> bool:
    return bool(_FLAGS["consumed"])


def mapping_validated(mark: bool = False) -> bool:
    """Has the batch packing of this scope been checked against the expected rows already?  ``mark`` records it."""
    if mark:
        _FLAGS["validated"] = True
    return bool(_FLAGS["validated"])


def assert_effective_overrides_consumed() -> None:
    if not _FLAGS["consumed"]:
        raise RuntimeError("TRIATTN_EFFECTIVE_OVERRIDES_NOT_CONSUMED:"
                           "runtime_overrides_activated_but_patched_input_prep_not_observed")


@contextmanager
def active_effective_input_overrides(overrides: EffectiveInputOverrides) -> Iterator[EffectiveInputOverrides]:
    global _ACTIVE
    _ACTIVE = overrides
    _FLAGS["consumed"] = _FLAGS["validated"] = False
    try:
        yield overrides
    finally:
        _ACTIVE = None
        _FLAGS["consumed"] = _FLAGS["validated"] = False


def execute_base_model_with_effective_overrides(*, base_runner: Any, state_store: Any, scheduler_output: Any,
                                                intermediate_tensors: Any = None, use_effective_overrides: bool = True,
                                                perf_out: Optional[dict] = None,
                                                override_scope: Callable = active_effective_input_overrides) -> Any:
    """Run the engine's ``execute_model``; inside ``override_scope`` when the step has overrides
    (``runtime/runner_output_bridge.py:18-83``)."""
    clock = time.perf_counter
    t0 = clock()
    overrides = None
    if use_effective_overrides:
        overrides = prepare_effective_input_overrides(base_runner=base_runner, state_store=state_store,
                                                      scheduler_output=scheduler_output)
    t1 = clock()
    if overrides is None or overrides.empty:
        output = base_runner.execute_model(scheduler_output=scheduler_output, intermediate_tensors=intermediate_tensors)
    else:
        with override_scope(overrides):
            output = base_runner.execute_model(scheduler_output=scheduler_output,
                                               intermediate_tensors=intermediate_tensors)
            # a runner with device-side request states must have gone through the patched input preparation
            if override_scope is active_effective_input_overrides and (
                    getattr(base_runner, "req_states", None) is not None
                    or os.environ.get("TRIATTN_DEBUG_ENABLE_V1_OVERRIDE_PATH", "0") == "1"):
                assert_effective_overrides_consumed()
    if isinstance(perf_out, dict):
        perf_out["override_prep_ms"] = (t1 - t0) * 1e3 if use_effective_overrides else 0.0
        perf_out["base_exec_ms"] = (clock() - t1) * 1e3
    return output


# ------------------------------------------------------------------------------------------------ events to the scheduler
def attach_execute_model_compression_events(*, output: Any, pending_events: list, scheduler_output: Any = None) -> tuple:
    """``(output, events still pending)``.  The events ride on the runner's output; with asynchronous scheduling
    ``execute_model`` returns None and they ride on the scheduler output instead (the same object comes back to
    the scheduler); an output that takes no attribute leaves them for ``sample_tokens``
    (``runtime/runner_output_bridge.py:86-133``)."""
    if output is None:
        if scheduler_output is not None and pending_events:
            setattr(scheduler_output, EVENTS_ATTR, pending_events)
            return output, []
        if pending_events:
            _log.warning("attach_events: no output and no scheduler output: %d events stay pending", len(pending_events))
        return output, pending_events
    try:
        setattr(output, EVENTS_ATTR, pending_events)
    except Exception:
        return output, pending_events
    return output, []


def attach_sample_tokens_compression_events(*, output: Any, pending_events: list) -> tuple:
    if output is None:
        return None, []
    setattr(output, EVENTS_ATTR, pending_events)
    return output, []


# ------------------------------------------------------------------------------------------------ the proxy
class TriAttentionModelRunner:
    """Wraps the engine's model runner; every attribute it does not define is the base runner's."""

    def __init__(self, base_runner: Any, config: Optional[TriAttentionRuntimeConfig] = None,
                 override_scope: Callable = active_effective_input_overrides,
                 install_runtime_input_patch: Optional[Callable[[], bool]] = None):
        self._base_runner = base_runner
        self.config = config or TriAttentionRuntimeConfig.from_env()
        self.state_store = RequestStateStore()
        setattr(base_runner, "_triattention_state_store", self.state_store)  # the hook reads the lengths kept here
        self.executor = _ra.RunnerHookCompressionExecutor(base_runner)
        self._last_step = 0
        self._logger = logging.getLogger(__name__)
        self._perf = TriAttentionPerfProfile.from_env(self._logger)
        self._pending_compression_events: list = []
        self._strict_no_downgrade = bool(self.config.enable_experimental_kv_compaction)
        self._allowed_strict_skip_reasons = set(STRICT_SKIP_REASONS)
        self._override_scope = override_scope
        self._install_runtime_input_patch = install_runtime_input_patch
        self._runtime_input_patch_installed = False

    def __getattr__(self, name: str) -> Any:
        return getattr(self._base_runner, name)

    def _ensure_runtime_input_patch_if_needed(self, needed: bool) -> None:
        """The engine-specific patch of the input preparation (given to the constructor) is installed the first time
        a step needs overrides on a runner that has the batch structures it patches."""
        if not needed or self._runtime_input_patch_installed or self._install_runtime_input_patch is None:
            return
        if getattr(self._base_runner, "req_states", None) is None and getattr(self._base_runner, "input_batch", None) is None:
            return
        if not self._install_runtime_input_patch():
            raise RuntimeError("TriAttention runtime requires gpu seq_len/slot_mapping patch when effective-length "
                               "overrides are active, but patch installation failed")
        self._runtime_input_patch_installed = True

    def execute_model(self, scheduler_output: Any, intermediate_tensors: Any = None) -> Any:
        perf_on = bool(getattr(self._perf, "enabled", False))
        clock = time.perf_counter
        t_start = clock()
        store, so = self.state_store, scheduler_output
        _ra.register_new_requests(state_store=store, scheduler_output=so, protect_prefill=bool(self.config.protect_prefill))
        _ra.cleanup_finished_requests(state_store=store, scheduler_output=so)
        _ra.mark_preemptions(state_store=store, scheduler_output=so)
        _ra.mark_resumed(state_store=store, scheduler_output=so)
        self._last_step, signals = _ra.consume_runner_signals(
            state_store=store, scheduler_output=so, last_step=self._last_step, logger=self._logger,
            log_decisions=bool(self.config.log_decisions))
        signals = supplement_worker_self_triggers(
            base_runner=self._base_runner, config=self.config, state_store=store, scheduler_output=so, signals=signals,
            last_step=self._last_step, logger=self._logger)
        t_state = clock()
        self._pending_compression_events = _ra.execute_runner_compression_actions(
            executor=self.executor, state_store=store, scheduler_output=so, signals=signals,
            strict_no_downgrade=self._strict_no_downgrade, allowed_strict_skip_reasons=self._allowed_strict_skip_reasons,
            logger=self._logger, log_decisions=bool(self.config.log_decisions))
        t_compress = clock()
        self._perf.record_compression_events(self._pending_compression_events)
        apply_worker_block_reclaim_events(base_runner=self._base_runner, events=self._pending_compression_events)
        trim_new_block_ids_for_compressed_reqs(base_runner=self._base_runner, state_store=store, scheduler_output=so,
                                               logger=self._logger)
        t_reclaim = clock()
        need = needs_effective_input_overrides(store, so)
        self._ensure_runtime_input_patch_if_needed(need)
        bridge: Optional[dict] = {} if perf_on else None
        output = execute_base_model_with_effective_overrides(
            base_runner=self._base_runner, state_store=store, scheduler_output=so,
            intermediate_tensors=intermediate_tensors, use_effective_overrides=need, perf_out=bridge,
            override_scope=self._override_scope)
        self._perf.record_model_output(output)
        self._perf.record_step(
            has_trigger=any(bool(s.should_compress) for s in signals.values()) if signals else False,
            uses_overrides=bool(need), t_state_ms=(t_state - t_start) * 1e3, t_compress_ms=(t_compress - t_state) * 1e3,
            t_reclaim_ms=(t_reclaim - t_compress) * 1e3,
            t_override_prep_ms=float((bridge or {}).get("override_prep_ms", 0.0)),
            t_base_exec_ms=float((bridge or {}).get("base_exec_ms", 0.0)), t_total_exec_ms=(clock() - t_start) * 1e3)
        output, self._pending_compression_events = attach_execute_model_compression_events(
            output=output, pending_events=self._pending_compression_events, scheduler_output=so)
        return output

    def sample_tokens(self, grammar_output: Any) -> Any:
        output = self._base_runner.sample_tokens(grammar_output)
        output, self._pending_compression_events = attach_sample_tokens_compression_events(
            output=output, pending_events=self._pending_compression_events)
        return output

    def snapshot_states(self) -> dict:
        return self.state_store.snapshot()


# ------------------------------------------------------------------------------------------------ worker wiring
# What the reference's worker subclass adds around the engine worker (runtime/worker.py:18-84): the engine's own
# model runner stays untouched through warm-up, graph capture and every step without a TriAttention signal; the
# first step that carries one installs the hook on it and wraps it in the proxy.
def backfill_model_path(worker: Any, config: TriAttentionRuntimeConfig) -> None:
    """The model directory (where the rotary configuration lives) from the engine's model config when the
    environment did not name one."""
    if config.model_path is not None:
        return
    path = getattr(getattr(worker, "model_config", None), "model", None)
    if isinstance(path, str) and path.strip():
        from pathlib import Path
        config.model_path = Path(path.strip())


def prepare_worker(worker: Any, config: Optional[TriAttentionRuntimeConfig] = None) -> None:
    """After the engine's ``init_device``: remember the configuration; install at once only when
    ``TRIATTN_DEBUG_EARLY_INSTALL_PROXY=1``."""
    if isinstance(getattr(worker, "model_runner", None), TriAttentionModelRunner):
        return
    worker._triattention_runtime_config = config or TriAttentionRuntimeConfig.from_env()
    backfill_model_path(worker, worker._triattention_runtime_config)
    worker._triattention_runner_proxy_installed = False
    if os.environ.get("TRIATTN_DEBUG_EARLY_INSTALL_PROXY", "0") == "1":
        ensure_runner_proxy(worker)


def ensure_runner_proxy(worker: Any, install_hook: Optional[Callable[..., None]] = None, **proxy_kwargs: Any) -> None:
    """Install the compression hook on ``worker.model_runner`` and replace it by the proxy (once)."""
    if getattr(worker, "_triattention_runner_proxy_installed", False):
        return
    if isinstance(worker.model_runner, TriAttentionModelRunner):
        worker._triattention_runner_proxy_installed = True
        return
    config = getattr(worker, "_triattention_runtime_config", None) or TriAttentionRuntimeConfig.from_env()
    backfill_model_path(worker, config)
    base_runner = worker.model_runner
    if install_hook is None:
        from .hook import install_runner_compression_hook as install_hook
    install_hook(base_runner=base_runner, config=config)
    worker.model_runner = TriAttentionModelRunner(base_runner, config, **proxy_kwargs)
    worker._triattention_runner_proxy_installed = True
    _log.info("TriAttention runner proxy installed: budget=%d divide_length=%d stats_path=%s model_path=%s "
              "protect_prefill=%s window_size=%s", config.kv_budget, config.divide_length, config.sparse_stats_path,
              config.model_path, config.protect_prefill, config.window_size)


def worker_execute_model(worker: Any, scheduler_output: Any, base_execute_model: Callable[[Any, Any], Any]) -> Any:
    """The worker's ``execute_model``: the proxy goes in with the first scheduler output that carries signals."""
    if getattr(scheduler_output, "triattention_signals", None):
        ensure_runner_proxy(worker)
    return base_execute_model(worker, scheduler_output)
