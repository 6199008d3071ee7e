"""Scheduler-side neighbours of the compression step: who asks for it and who frees what it left over.

The reference's additions to the engine-core process, kept free of any engine import (they work on the
attributes the reference reads, so the reference's scheduler subclass or its patches can bind them as they are):

* :class:`CompressionPlanner` - the trigger: cache length >= budget + divide_length (+ the prompt when it is
  protected outside the budget), or KV-pool pressure with hysteresis (``runtime/planner.py:9-62``).  Its
  ``CompressionSignal`` is what the worker-side driver consumes.
* :class:`EffectiveCacheLenTracker` - cache length of a request as the scheduler sees it: the engine's monotonic
  ``num_computed_tokens`` until the first compression, afterwards the compacted length plus the tokens computed
  since (``runtime/effective_len_tracker.py:6-68``).
* the request attributes that keep slot allocation in step after blocks were given back
  (``runtime/kv_allocation_sync.py:8-94``).
* :func:`apply_compression_events` - the block-pool side of the reclaim: for every applied compression of a step,
  shrink the request's block list of each KV-cache group to the prefix the worker kept and return the old tail
  blocks to the pool, with the consistency checks and the batch-queue fall-backs of
  ``runtime/scheduler.py:29-52,338-564``.
* the scheduler's step around the engine's own ``schedule`` / ``update_from_output``: :func:`schedule_with_signals`
  (allocation markers, the token cap of a small pool, prompt lengths, the sparse signal dictionary) and
  :func:`update_from_output_with_events` (``runtime/scheduler.py:123-336,566-595``,
  ``runtime/integration_monkeypatch.py:89-216``).
"""
from __future__ import annotations

import logging
from typing import Any, Iterable, Optional

from .config import TriAttentionRuntimeConfig
from .signals import CompressionSignal

EFFECTIVE_KV_OFFSET_ATTR = "_triattention_effective_kv_offset"
EFFECTIVE_NUM_COMPUTED_ATTR = "_triattention_effective_num_computed_tokens"

_log = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------------ trigger
class CompressionPlanner:
    """One decision per request and step.  The KV-pool trigger latches: armed at ``kv_usage_trigger``, released
    only at ``kv_usage_release``, and it wins the ``reason`` when both triggers fire."""

    def __init__(self, config: TriAttentionRuntimeConfig) -> None:
        self.config = config
        self._kv_pressure_armed = False

    def _pool_pressure(self, kv_usage: Optional[float]) -> bool:
        cfg = self.config
        if kv_usage is None or not cfg.enable_kv_usage_trigger:
            return False  # the latch keeps its state while the trigger is not consulted
        if kv_usage >= cfg.kv_usage_trigger:
            self._kv_pressure_armed = True
        elif kv_usage <= cfg.kv_usage_release:
            self._kv_pressure_armed = False
        return self._kv_pressure_armed

    def length_threshold(self, prefill_len: int) -> int:
        cfg = self.config
        extra = max(prefill_len, 0) if (cfg.protect_prefill and not cfg.include_prefill_in_budget) else 0
        return cfg.kv_budget + cfg.divide_length + extra

    def build_signal(self, req_id: str, estimated_cache_len: int, prefill_len: int, step: int,
                     kv_usage: Optional[float] = None, scheduled_tokens: int = 1) -> CompressionSignal:
        by_length = estimated_cache_len >= self.length_threshold(prefill_len)
        by_pool = self._pool_pressure(kv_usage)
        reason = "kv_usage_threshold" if by_pool else ("length_threshold" if by_length else "none")
        return CompressionSignal(
            req_id=req_id, should_compress=by_length or by_pool, reason=reason, estimated_cache_len=estimated_cache_len,
            step=step, kv_usage=kv_usage, protect_prefill=self.config.protect_prefill, prefill_len=prefill_len,
            scheduled_tokens=max(1, int(scheduled_tokens)))


# ------------------------------------------------------------------------------------------------ lengths
class EffectiveCacheLenTracker:
    """``observe_num_computed`` returns the length the trigger should test.  A request without a compression so
    far has no entry in ``_effective_len`` and simply reports the engine's counter."""

    def __init__(self) -> None:
        self._effective_len: dict = {}
        self._last_num_computed: dict = {}

    def reset_request(self, req_id: str, num_computed_tokens: int) -> None:
        self._effective_len.pop(req_id, None)
        self._last_num_computed[req_id] = max(0, int(num_computed_tokens))

    def remove_request(self, req_id: str) -> None:
        self._effective_len.pop(req_id, None)
        self._last_num_computed.pop(req_id, None)

    def observe_num_computed(self, req_id: str, num_computed_tokens: int) -> int:
        now = max(0, int(num_computed_tokens))
        effective = self._effective_len.get(req_id)
        if effective is None:
            self._last_num_computed[req_id] = now
            return now
        before = self._last_num_computed.get(req_id, now)
        # forward progress is appended; a counter that went backwards (rollback) can only cap the length
        effective = effective + (now - before) if now >= before else min(effective, now)
        effective = max(0, effective)
        self._effective_len[req_id] = effective
        self._last_num_computed[req_id] = now
        return effective

    def apply_compression(self, req_id: str, cache_len_after: int, num_computed_tokens: int) -> None:
        self._effective_len[req_id] = max(0, int(cache_len_after))
        self._last_num_computed[req_id] = max(0, int(num_computed_tokens))

    def snapshot(self) -> dict:
        ids = set(self._effective_len) | set(self._last_num_computed)
        return {r: (self._effective_len.get(r, -1), self._last_num_computed.get(r)) for r in ids}

    def has_effective_len_override(self, req_id: str) -> bool:
        return req_id in self._effective_len

    def has_any_effective_len_overrides(self) -> bool:
        return bool(self._effective_len)


# ------------------------------------------------------------------------------------------------ allocation sync
def _count(value: Any) -> Optional[int]:
    try:
        return max(0, int(value))
    except (TypeError, ValueError):
        return None


def _drop_attr(obj: Any, name: str) -> None:
    if hasattr(obj, name):
        try:
            delattr(obj, name)
        except Exception:
            setattr(obj, name, None)


def clear_request_allocation_sync_state(request: Any) -> None:
    if request is None:
        return
    for name in (EFFECTIVE_KV_OFFSET_ATTR, EFFECTIVE_NUM_COMPUTED_ATTR):
        try:
            _drop_attr(request, name)
        except Exception:
            continue


def update_request_effective_kv_offset(*, request: Any, cache_len_after: int) -> Optional[int]:
    """Remember on the request how far its logical progress is ahead of what its blocks hold (0 clears it)."""
    if request is None:
        return None
    logical, effective = _count(getattr(request, "num_computed_tokens", None)), _count(cache_len_after)
    if logical is None or effective is None:
        return None
    offset = logical - min(effective, logical)
    if offset <= 0:
        _drop_attr(request, EFFECTIVE_KV_OFFSET_ATTR)
        return 0
    setattr(request, EFFECTIVE_KV_OFFSET_ATTR, offset)
    return offset


def prepare_request_effective_num_computed(request: Any) -> Optional[int]:
    """Before a scheduling step: logical progress minus the remembered offset, as the marker the allocation patch
    reads; a request that restarted (progress 0 or behind the offset) loses both attributes."""
    if request is None:
        return None
    logical = _count(getattr(request, "num_computed_tokens", None))
    if logical is None:
        return None
    offset = _count(getattr(request, EFFECTIVE_KV_OFFSET_ATTR, None))
    if not offset:
        _drop_attr(request, EFFECTIVE_NUM_COMPUTED_ATTR)
        return None
    if logical == 0 or logical < offset:
        clear_request_allocation_sync_state(request)
        return None
    setattr(request, EFFECTIVE_NUM_COMPUTED_ATTR, logical - offset)
    return logical - offset


def resolve_request_effective_num_computed(request: Any) -> Optional[int]:
    if request is None:
        return None
    logical = _count(getattr(request, "num_computed_tokens", None))
    effective = _count(getattr(request, EFFECTIVE_NUM_COMPUTED_ATTR, None))
    if logical is None or effective is None or effective > logical:
        return None
    return effective


# ------------------------------------------------------------------------------------------------ block-pool reclaim
def free_reclaimed_blocks(manager: Any, removed_blocks: list) -> bool:
    """Give ``removed_blocks`` back to the manager's pool, last block first, after dropping the prefix-cache identity
    of those that carry a hash.  False when there was nothing to free or no pool to free into."""
    if not removed_blocks:
        return False
    pool = getattr(manager, "block_pool", None)
    evict = getattr(pool, "_maybe_evict_cached_block", None) if pool is not None else None
    if callable(evict):
        for block in removed_blocks:
            if block is not None and getattr(block, "block_hash", None) is not None:
                evict(block)
    if pool is None:
        return False
    pool.free_blocks(reversed(removed_blocks))
    return True


def _cap_cached_count(manager: Any, req_id: Any, n_blocks: int) -> None:
    if req_id in manager.num_cached_block:
        manager.num_cached_block[req_id] = min(manager.num_cached_block[req_id], n_blocks)


def _truncate_to(manager: Any, req_id: Any, n_blocks: int) -> bool:
    """No explicit payload for this group: keep the first ``n_blocks`` blocks of the request, free the rest."""
    blocks = manager.req_to_blocks.get(req_id)
    if not blocks or n_blocks >= len(blocks):
        return False
    manager.req_to_blocks[req_id] = blocks[:n_blocks]
    _cap_cached_count(manager, req_id, n_blocks)
    return free_reclaimed_blocks(manager, blocks[n_blocks:])


def _apply_group_payload(manager: Any, req_id: Any, gid: int, group: dict, ids_after: list, required: int,
                         must_reach_required: bool) -> bool:
    blocks = manager.req_to_blocks[req_id]
    have = [blk.block_id for blk in blocks]
    kept = len(ids_after)
    if kept > len(have):
        raise RuntimeError(f"TriAttention block reclaim invalid length: req={req_id} gid={gid} kept_len={kept} "
                           f"curr_len={len(have)}")
    if len(set(ids_after)) != kept:
        raise RuntimeError(f"TriAttention block reclaim contains duplicate block ids: req={req_id} gid={gid} "
                           f"block_ids_after={ids_after}")
    if have[:kept] != ids_after:
        raise RuntimeError(f"TriAttention block reclaim prefix mismatch: req={req_id} gid={gid} "
                           f"expected_prefix={have[:kept]} actual_after={ids_after}")
    if must_reach_required and kept != required:
        raise RuntimeError(f"TriAttention block reclaim insufficient shrink: req={req_id} gid={gid} kept_len={kept} "
                           f"required_blocks={required}")
    # Blocks appended after the hook ran (same step, asynchronous scheduling) are not in ``block_ids_before``:
    # they stay, behind the kept prefix; only the old tail goes back to the pool.
    before = group.get("block_ids_before")
    n_old = len(before) if isinstance(before, list) else len(blocks)
    old_tail, appended = list(blocks[kept:n_old]), list(blocks[n_old:])
    manager.req_to_blocks[req_id] = list(blocks[:kept]) + appended
    _cap_cached_count(manager, req_id, kept + len(appended))
    if not old_tail:
        return False
    _log.info("TriAttention scheduler FREE_BLOCKS: req=%s gid=%d freed=%d kept=%d new=%d", req_id, gid, len(old_tail),
              kept, len(appended))
    return free_reclaimed_blocks(manager, old_tail)


def apply_compression_events(scheduler: Any, compression_events: Iterable[dict]) -> None:
    """Consume the events the worker attached to its output (``execute_runner_compression_actions``).

    ``scheduler`` offers ``kv_cache_manager.coordinator.single_type_managers`` (each with ``req_to_blocks``,
    ``num_cached_block``, ``block_pool``), ``block_size``, ``requests``, ``_effective_len_tracker`` and
    ``triattention_config``.  A group the event does not describe is shrunk to ``ceil(cache_len_after / block_size)``
    blocks when the step scheduled a single token (the worker had truncated it in an earlier step of the batch
    queue); during a chunked prefill such a group is left alone, because blocks appended since cannot be told from
    old ones.  Inconsistent payloads raise; see the four messages above.
    """
    managers = getattr(getattr(scheduler.kv_cache_manager, "coordinator", None), "single_type_managers", None)
    indexable = isinstance(managers, (list, tuple))
    block_size = int(getattr(scheduler, "block_size", 1))
    if block_size <= 0:
        block_size = 1
    cfg = scheduler.triattention_config
    for event in compression_events:
        if event.get("status") != "applied" or event.get("req_id") is None:
            continue
        req_id = event["req_id"]
        int(event.get("step", -1))  # a malformed step is an error here as well
        after = event.get("cache_len_after")
        if not isinstance(after, int):
            continue
        request = scheduler.requests.get(req_id)
        if request is None:
            continue
        scheduler._effective_len_tracker.apply_compression(req_id=req_id, cache_len_after=after,
                                                           num_computed_tokens=request.num_computed_tokens)
        if not cfg.enable_experimental_block_reclaim:
            continue
        required = (after + block_size - 1) // block_size if after > 0 else 0
        single_token_step = int(event.get("scheduled_tokens", 1)) <= 1
        oversized = set()
        if indexable:
            for gid, manager in enumerate(managers):
                blocks = manager.req_to_blocks.get(req_id)
                if blocks and required < len(blocks):
                    oversized.add(gid)
        payload = event.get("block_reclaim")
        groups = payload.get("groups") if isinstance(payload, dict) else None
        freed = False
        described = set()
        if isinstance(groups, list):
            if not indexable:
                continue
            for group in groups:
                if not isinstance(group, dict):
                    continue
                gid, ids_after = group.get("gid"), group.get("block_ids_after")
                if not isinstance(gid, int) or not 0 <= gid < len(managers) or not isinstance(ids_after, list):
                    continue
                if not all(isinstance(x, int) for x in ids_after) or not managers[gid].req_to_blocks.get(req_id):
                    continue
                described.add(gid)
                must = bool(getattr(cfg, "require_physical_reclaim", False)) and gid in oversized
                if _apply_group_payload(managers[gid], req_id, gid, group, ids_after, required, must):
                    freed = True
        left_over = oversized - described
        if left_over and not single_token_step:
            _log.info("TriAttention block reclaim: skipping synthesized reclaim for gids %s during prefill "
                      "(scheduled_tokens=%s) req=%s", sorted(left_over), event.get("scheduled_tokens", 1), req_id)
        elif left_over and indexable:
            for gid in sorted(left_over):
                if _truncate_to(managers[gid], req_id, required):
                    freed = True
        if freed:
            update_request_effective_kv_offset(request=request, cache_len_after=after)


# ------------------------------------------------------------------------------------------------ the scheduler's step
# What the reference adds around the engine scheduler's ``schedule`` and ``update_from_output``
# (runtime/scheduler.py:84-336,566-595 and the patched forms in runtime/integration_monkeypatch.py:89-216), as
# functions over a scheduler object that carries the six attributes set by :func:`attach_scheduler_state`.
def attach_scheduler_state(scheduler: Any, config: Optional[TriAttentionRuntimeConfig] = None) -> None:
    cfg = config or TriAttentionRuntimeConfig.from_env()
    scheduler.triattention_config = cfg
    scheduler._planner = CompressionPlanner(cfg)
    scheduler._effective_len_tracker = EffectiveCacheLenTracker()
    scheduler._prefill_lens = {}
    scheduler._length_threshold_cache = {}
    scheduler._triattention_step = 0


def _prompt_len(request_like: Any) -> int:
    from .runner_actions import full_prefill_len  # the same "largest of the fields that exist" rule on both sides
    return full_prefill_len(request_like)


def _threshold_for(cfg: Any, prefill_len: int) -> int:
    extra = max(0, int(prefill_len)) if (cfg.protect_prefill and not cfg.include_prefill_in_budget) else 0
    return cfg.kv_budget + cfg.divide_length + extra


def _known_prefill_len(scheduler: Any, req_id: Any) -> int:
    if req_id in scheduler._prefill_lens:
        return scheduler._prefill_lens[req_id]
    request = scheduler.requests.get(req_id)
    return 0 if request is None else request.num_prompt_tokens


def _remember_prefill_len(scheduler: Any, req_id: Any, prefill_len: int) -> None:
    scheduler._prefill_lens[req_id] = prefill_len
    scheduler._length_threshold_cache[req_id] = _threshold_for(scheduler.triattention_config, prefill_len)


def sync_prefill_lens(scheduler: Any, scheduler_output: Any) -> None:
    """Prompt lengths and thresholds of arriving requests (the tracker is reset only at a request's FIRST
    appearance: a chunked prefill lists it again), forgotten for finished ones, recovered for resumed ones."""
    for new_req in scheduler_output.scheduled_new_reqs:
        if new_req.req_id not in scheduler._prefill_lens:
            scheduler._effective_len_tracker.reset_request(new_req.req_id, new_req.num_computed_tokens)
        _remember_prefill_len(scheduler, new_req.req_id, _prompt_len(new_req))
    for req_id in scheduler_output.finished_req_ids:
        request = scheduler.requests.get(req_id)
        if request is not None:
            clear_request_allocation_sync_state(request)
        scheduler._prefill_lens.pop(req_id, None)
        scheduler._length_threshold_cache.pop(req_id, None)
        scheduler._effective_len_tracker.remove_request(req_id)
    cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
    resumed = [] if cached is None else getattr(cached, "resumed_req_ids", None)
    if resumed is None:
        resumed = getattr(cached, "req_ids", []) or []
    for req_id in resumed:
        if req_id not in scheduler._prefill_lens:
            _remember_prefill_len(scheduler, req_id, _known_prefill_len(scheduler, req_id))


def build_signals(scheduler: Any, scheduler_output: Any) -> dict:
    """Signals of the step, sparse: only requests that trigger now or have been compressed before (those still need
    their effective length on the worker).  An uncompressed request below its threshold costs one dictionary lookup
    and one comparison."""
    from .effective_overrides import scheduled_token_items

    cfg = scheduler.triattention_config
    by_pool = bool(cfg.enable_kv_usage_trigger)
    kv_usage = scheduler.kv_cache_manager.usage if by_pool else None
    off = bool(cfg.disable_compression)
    tracker = scheduler._effective_len_tracker
    signals: dict = {}
    for _key, req_id, scheduled in scheduled_token_items(scheduler_output):
        request = scheduler.requests.get(req_id)
        if request is None:
            continue
        compressed = tracker.has_effective_len_override(req_id)
        base = (tracker.observe_num_computed(req_id=req_id, num_computed_tokens=request.num_computed_tokens)
                if compressed else request.num_computed_tokens)
        estimate = base + scheduled
        if not compressed and not by_pool:
            if off:
                continue
            threshold = scheduler._length_threshold_cache.get(req_id)
            if threshold is None:
                _remember_prefill_len(scheduler, req_id, _known_prefill_len(scheduler, req_id))
                threshold = scheduler._length_threshold_cache[req_id]
            if estimate < threshold:
                continue
        prefill_len = scheduler._prefill_lens.get(req_id)
        if prefill_len is None:
            prefill_len = _known_prefill_len(scheduler, req_id)
            _remember_prefill_len(scheduler, req_id, prefill_len)
        signal = scheduler._planner.build_signal(req_id=req_id, estimated_cache_len=estimate, prefill_len=prefill_len,
                                                 step=scheduler._triattention_step, kv_usage=kv_usage,
                                                 scheduled_tokens=scheduled)
        if signal.should_compress or compressed:
            signals[req_id] = signal
    return signals


def max_chunk_for_compression(scheduler: Any, cfg: Any) -> Optional[int]:
    """Largest number of tokens a step may schedule so that budget + chunk still fits the physical pool (minus one
    block of slack); None when no cap applies."""
    pool = getattr(getattr(scheduler, "kv_cache_manager", None), "block_pool", None)
    total = getattr(pool, "num_gpu_blocks", 0) if pool is not None else 0
    if pool is None or total <= 0:
        return None
    block_size = int(getattr(scheduler, "block_size", 16) or 16)
    headroom = total * block_size - cfg.kv_budget
    return max(1, headroom - block_size) if headroom > 0 else None


def schedule_with_signals(scheduler: Any, base_schedule: Any) -> Any:
    """``base_schedule(scheduler)`` with the allocation markers refreshed before it, the step's token cap lowered
    around it when the pool is small, and ``triattention_step`` / ``triattention_signals`` attached to its result."""
    running = getattr(scheduler, "running", None)
    if isinstance(running, list):
        for request in running:
            prepare_request_effective_num_computed(request)
    cfg = getattr(scheduler, "triattention_config", None)
    saved_cap = None
    if cfg and not cfg.disable_compression:
        cap = max_chunk_for_compression(scheduler, cfg)
        current = getattr(scheduler, "max_num_scheduled_tokens", None)
        if cap is not None and current is not None and cap < current:
            saved_cap, scheduler.max_num_scheduled_tokens = current, cap
    scheduler_output = base_schedule(scheduler)
    if saved_cap is not None:
        scheduler.max_num_scheduled_tokens = saved_cap
    if cfg is None:
        return scheduler_output
    scheduler._triattention_step += 1
    sync_prefill_lens(scheduler, scheduler_output)
    idle = (cfg.disable_compression and not cfg.enable_kv_usage_trigger
            and not scheduler._effective_len_tracker.has_any_effective_len_overrides())
    scheduler_output.triattention_step = scheduler._triattention_step
    scheduler_output.triattention_signals = {} if idle else build_signals(scheduler, scheduler_output)
    return scheduler_output


def update_from_output_with_events(scheduler: Any, scheduler_output: Any, model_runner_output: Any,
                                   base_update: Any) -> Any:
    """``base_update(scheduler, scheduler_output, model_runner_output)``, then the compression events of the step -
    from the runner's output, else (asynchronous scheduling) from the scheduler output - are applied and the pool
    usage in the returned statistics is brought up to date."""
    outputs = base_update(scheduler, scheduler_output, model_runner_output)
    if getattr(scheduler, "triattention_config", None) is None:
        return outputs
    events = getattr(model_runner_output, "triattention_compression_events", None) or \
        getattr(scheduler_output, "triattention_compression_events", None)
    if events:
        apply_compression_events(scheduler, events)
        if isinstance(outputs, dict):
            usage = float(scheduler.kv_cache_manager.usage)
            for engine_output in outputs.values():
                stats = getattr(engine_output, "scheduler_stats", None)
                if stats is not None:
                    stats.kv_cache_usage = usage
    for req_id in scheduler_output.finished_req_ids:
        scheduler._prefill_lens.pop(req_id, None)
        scheduler._length_threshold_cache.pop(req_id, None)
        scheduler._effective_len_tracker.remove_request(req_id)
    return outputs


# ------------------------------------------------------------------------------------------------ slot allocation
def allocate_slots_with_effective_length(manager: Any, request: Any, num_new_tokens: int, *args: Any,
                                         base_allocate: Any, **kwargs: Any) -> Any:
    """``base_allocate(manager, request, num_new_tokens, ...)`` - the engine's ``KVCacheManager.allocate_slots`` -
    seeing the request's EFFECTIVE progress.

    A request whose blocks were given back holds fewer tokens than its logical ``num_computed_tokens``; for the
    duration of the call the counter is replaced by the effective value (and put back whatever happens), so that
    the engine allocates for the cache as it is.  The compacted layout no longer matches the engine's prefix-hash
    chain, so the call also asks it not to commit prefix-cache hashes (``delay_cache_blocks=True``).  Requests
    without a reclaim go straight through (``runtime/integration_monkeypatch.py:243-284``)."""
    prepare_request_effective_num_computed(request)  # waiting (preempted) requests are not refreshed by the schedule step
    effective = resolve_request_effective_num_computed(request)
    logical = getattr(request, "num_computed_tokens", None)
    if effective is None or not isinstance(logical, int) or effective >= logical:
        return base_allocate(manager, request, num_new_tokens, *args, **kwargs)
    request.num_computed_tokens = int(effective)
    try:
        return base_allocate(manager, request, num_new_tokens, *args, **{**kwargs, "delay_cache_blocks": True})
    finally:
        request.num_computed_tokens = logical


def scheduler_output_has_compression_boundary(scheduler_output: Any) -> bool:
    """Does this step carry a trigger?  An asynchronous engine must not let its batch queue run ahead of such a step
    (``runtime/integration_monkeypatch.py:287-291``)."""
    signals = getattr(scheduler_output, "triattention_signals", None)
    if not isinstance(signals, dict) or not signals:
        return False
    return any(bool(getattr(sig, "should_compress", False)) for sig in signals.values())


def batch_queue_has_pending_compression_boundary(batch_queue: Any) -> bool:
    """Is a step marked ``_triattention_force_boundary_sync`` still waiting in the engine's batch queue (entries
    ``(future, scheduler_output, ...)``)?  (``runtime/integration_monkeypatch.py:294-307``)"""
    if batch_queue is None:
        return False
    try:
        entries = list(batch_queue)
    except Exception:
        return False
    return any(isinstance(e, tuple) and len(e) >= 2 and bool(getattr(e[1], "_triattention_force_boundary_sync", False))
               for e in entries)
