"""Duck-typed views of a request inside the serving engine's model runner.

Covers the runner layouts the reference supports (runtime/hook_preflight.py:118-210,
runtime/runner_struct_compat.py:59-135, runtime/request_key_compat.py): ``base_runner.requests[req_id]``
with ``block_ids`` / ``num_computed_tokens``; the newer ``block_tables`` + ``req_states`` / ``input_batch``
arrays; and, for brand-new requests, the scheduler output itself.  Setting ``block_ids`` on a view is the
block-table rewrite after compaction.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


def _req_id_of(key: Any):
    if isinstance(key, (str, int)):
        return key
    for attr in ("request_id", "req_id"):
        v = getattr(key, attr, None)
        if isinstance(v, (str, int)):
            return v
    return None


def scheduled_tokens_for_req(scheduler_output: Any, req_id) -> int:
    """Tokens scheduled for ``req_id`` in this step, at least 1 (hook_runtime_context.py:56-74)."""
    sched = getattr(scheduler_output, "num_scheduled_tokens", None)
    if isinstance(sched, dict):
        for key, value in sched.items():
            if _req_id_of(key) == req_id:
                try:
                    return max(1, int(value))
                except (TypeError, ValueError):
                    break
    return 1


@dataclass
class SchedulerOutputRequestStateView:
    req_id: str
    num_computed_tokens: int
    block_ids: Any


@dataclass
class MergedRequestStateView:
    """Runner state whose ``num_computed_tokens`` lags the scheduler's: take the larger value."""

    base_req_state: Any
    overridden_num_computed_tokens: int
    fallback_block_ids: Any = None

    @property
    def num_computed_tokens(self) -> int:
        return int(self.overridden_num_computed_tokens)

    @property
    def block_ids(self) -> Any:
        ids = getattr(self.base_req_state, "block_ids", None)
        return ids if ids is not None else self.fallback_block_ids

    @block_ids.setter
    def block_ids(self, value: Any) -> None:
        setattr(self.base_req_state, "block_ids", value)


@dataclass
class CompatRequestStateView:
    """Request view over ``base_runner.block_tables`` / ``req_states`` / ``input_batch`` arrays."""

    base_runner: Any
    req_id: str
    req_index: int
    requests_state: Optional[Any] = None

    @property
    def num_computed_tokens(self) -> int:
        rs = getattr(self.base_runner, "req_states", None)
        gpu = getattr(getattr(rs, "num_computed_tokens", None), "gpu", None)
        if torch.is_tensor(gpu):
            return int(gpu[self.req_index].item())
        cpu = getattr(getattr(self.base_runner, "input_batch", None), "num_computed_tokens_cpu", None)
        if cpu is not None:
            try:
                return int(cpu[self.req_index])
            except Exception:
                pass
        return 0

    @property
    def block_ids(self):
        bts = getattr(self.base_runner, "block_tables", None)
        tables = getattr(bts, "block_tables", None) if bts is not None else None
        counts = getattr(getattr(bts, "num_blocks", None), "np", None) if bts is not None else None
        if isinstance(tables, list) and counts is not None:
            out, ok = [], True
            for gid, table in enumerate(tables):
                try:
                    n = int(counts[gid, self.req_index])
                except Exception:
                    ok = False
                    break
                if n <= 0:
                    out.append([])
                    continue
                row = getattr(table, "gpu", None)
                if not torch.is_tensor(row):
                    ok = False
                    break
                out.append([int(x) for x in row[self.req_index, :n].tolist()])
            if ok and any(out):
                return tuple(out)
        fb = getattr(self.requests_state, "block_ids", None)
        if isinstance(fb, (list, tuple)):
            return tuple([int(x) for x in g] if isinstance(g, (list, tuple)) else [] for g in fb)
        return None

    @block_ids.setter
    def block_ids(self, new_ids) -> None:
        if not isinstance(new_ids, (list, tuple)):
            raise TypeError("block_ids must be a list/tuple by group")
        norm = tuple([int(x) for x in g] if isinstance(g, (list, tuple)) else [] for g in new_ids)
        bts = getattr(self.base_runner, "block_tables", None)
        if bts is not None:
            bts.append_block_ids(self.req_index, norm, overwrite=True)
            bts.apply_staged_writes()
        if self.requests_state is not None:
            setattr(self.requests_state, "block_ids", norm)


def _req_index(base_runner: Any, req_id) -> Optional[int]:
    """Row of the request in the runner's batch arrays: req_states, then input_batch, then its req_ids list."""
    input_batch = getattr(base_runner, "input_batch", None)
    for holder in (getattr(base_runner, "req_states", None), input_batch):
        table = getattr(holder, "req_id_to_index", None) if holder is not None else None
        if isinstance(table, dict) and isinstance(table.get(req_id), int):
            return int(table[req_id])
    if input_batch is not None:
        ids = getattr(input_batch, "req_ids", None)
        try:
            ids = ids() if callable(ids) else ids
        except Exception:
            ids = None
        if not isinstance(ids, list):
            ids = getattr(input_batch, "_req_ids", None)
        if isinstance(ids, list) and req_id in ids:
            return ids.index(req_id)
    return None


def resolve_request_state_view(base_runner: Any, req_id):
    """(state view, source label) or (None, 'none')."""
    requests = getattr(base_runner, "requests", None)
    state = requests.get(req_id) if isinstance(requests, dict) else None
    idx = _req_index(base_runner, req_id)
    if idx is not None:
        return CompatRequestStateView(base_runner, req_id, idx, state), "batch_arrays"
    if state is not None:
        return state, "requests"
    return None, "none"


def _scheduler_output_view(scheduler_output: Any, req_id):
    new_reqs = getattr(scheduler_output, "scheduled_new_reqs", None)
    if isinstance(new_reqs, list):
        for nr in new_reqs:
            if getattr(nr, "req_id", None) != req_id or getattr(nr, "block_ids", None) is None:
                continue
            lens = []
            for attr in ("prompt_token_ids", "prefill_token_ids"):
                v = getattr(nr, attr, None)
                if v is not None:
                    try:
                        lens.append(len(v))
                    except Exception:
                        pass
            for attr in ("prompt_token_ids_len", "num_prompt_tokens"):
                v = getattr(nr, attr, None)
                if v is not None:
                    try:
                        lens.append(int(v))
                    except (TypeError, ValueError):
                        pass
            return SchedulerOutputRequestStateView(req_id, int(max(lens, default=0)), nr.block_ids)
    cached = getattr(scheduler_output, "scheduled_cached_reqs", None)
    ids = getattr(cached, "req_ids", None)
    computed = getattr(cached, "num_computed_tokens", None)
    if isinstance(ids, list) and isinstance(computed, list):
        for i, rid in enumerate(ids):
            if rid == req_id and i < len(computed):
                try:
                    return SchedulerOutputRequestStateView(req_id, int(computed[i]), None)
                except Exception:
                    continue
    return None


@dataclass(frozen=True)
class HookRequestContext:
    req_state: Any
    req_runtime_state: Any


def resolve_hook_request_context(*, base_runner: Any, req_id, scheduler_output: Any = None):
    """Request state + per-request runtime state, or ``{"applied": False, "reason": "req_state_not_found"}``."""
    state, _source = resolve_request_state_view(base_runner, req_id)
    so_view = _scheduler_output_view(scheduler_output, req_id) if scheduler_output is not None else None
    if state is not None and so_view is not None:
        try:
            mine = int(getattr(state, "num_computed_tokens", 0) or 0)
            theirs = int(getattr(so_view, "num_computed_tokens", 0) or 0)
            if theirs > mine:
                state = MergedRequestStateView(state, theirs, getattr(so_view, "block_ids", None))
        except Exception:
            pass
    if state is None:
        state = so_view
    if state is None:
        return {"applied": False, "reason": "req_state_not_found"}
    store = getattr(base_runner, "_triattention_state_store", None)
    runtime_state = store.get(req_id) if store is not None and hasattr(store, "get") else None
    return HookRequestContext(state, runtime_state)
