"""Scripted inputs for the worker-side action driver, shared by the fixture generator (which runs the reference's
``execute_runner_compression_actions`` on them) and by the test (which runs this package's driver on them)."""
from __future__ import annotations

import logging
import types


class ScriptedExecutor:
    """Answers ``execute`` from a script {req_id: result dict | bool | ("raise", type name, message)}."""

    def __init__(self, script: dict, result_cls, with_batch: bool = False):
        self._script, self._result_cls = script, result_cls
        self.calls = []
        if with_batch:
            self.execute_batch = self._execute_batch

    def _one(self, req_id):
        self.calls.append(req_id)
        spec = self._script[req_id]
        if isinstance(spec, (list, tuple)) and spec and spec[0] == "raise":
            raise {"ValueError": ValueError, "RuntimeError": RuntimeError}[spec[1]](spec[2])
        if isinstance(spec, bool):
            return self._result_cls(applied=spec, reason="applied" if spec else "runner_hook_rejected")
        d = dict(spec)
        return self._result_cls(applied=bool(d.get("applied", False)), reason=str(d.get("reason", "runner_hook_result")),
                                cache_len_after=d.get("cache_len_after"), details=d)

    def execute(self, req_id, signal, scheduler_output):
        return self._one(req_id)

    def _execute_batch(self, requests, scheduler_output):
        return {req_id: self._one(req_id) for req_id, _ in requests}


class RecordingStore:
    """State store that remembers every bookkeeping call."""

    def __init__(self, states: dict):
        self._states = {k: types.SimpleNamespace(**v) for k, v in states.items()}
        self.calls = []

    def get(self, req_id):
        return self._states.get(req_id)

    def mark_compressed(self, **kw):
        self.calls.append(["mark_compressed", kw])

    def mark_compression_skipped(self, **kw):
        self.calls.append(["mark_compression_skipped", kw])


def _sig(req_id, step, should=True, est=3000, sched=1, prefill=0):
    return dict(req_id=req_id, should_compress=should, reason="length_threshold", estimated_cache_len=est, step=step,
                kv_usage=None, protect_prefill=False, prefill_len=prefill, scheduled_tokens=sched)


APPLIED = {"applied": True, "reason": "kv_compacted:per_head", "cache_len_after": 2048,
           "effective_tokens_before": 2176, "budget_total": 2048, "reclaimed_block_count": 8,
           "recent_unabsorbed_tokens": 128,
           "block_reclaim": {"mode": "truncate_tail", "groups": [{"gid": 0, "block_ids_before": [1, 2, 3],
                                                                  "block_ids_after": [1, 2]}]}}
SKIPPED = {"applied": False, "reason": "under_budget", "cache_len_after": 1900}


def scenarios() -> list:
    so = {"req_ids": ["a", "c"], "num_computed_tokens": [2175, 900]}
    return [
        dict(name="mixed", strict=False, allowed=[], scheduler=so,
             signals=[_sig("a", 7), _sig("b", 7, should=False), _sig("c", 7), _sig("d", 7), _sig("e", 7, sched=512)],
             script={"a": APPLIED, "c": SKIPPED, "d": APPLIED, "e": {"applied": True, "reason": "kv_compacted:per_head"}},
             states={"d": dict(last_compression_step=6, compression_count=2, current_cache_len=2050),
                     "e": dict(last_compression_step=6, compression_count=1, current_cache_len=2600)}),
        dict(name="bool_results", strict=False, allowed=[], scheduler=None,
             signals=[_sig("a", 3), _sig("b", 3)], script={"a": True, "b": False}, states={}),
        dict(name="soft_exception", strict=False, allowed=[], scheduler=None,
             signals=[_sig("a", 4), _sig("b", 4)], script={"a": ("raise", "ValueError", "boom"), "b": APPLIED}, states={}),
        dict(name="strict_exception", strict=True, allowed=["under_budget"], scheduler=None,
             signals=[_sig("a", 5), _sig("b", 5)], script={"a": APPLIED, "b": ("raise", "ValueError", "boom")}, states={}),
        dict(name="strict_unexpected_skip", strict=True, allowed=["prefill_exceeds_budget"], scheduler=None,
             signals=[_sig("a", 6), _sig("b", 6)], script={"a": SKIPPED, "b": APPLIED}, states={}),
        dict(name="strict_allowed_skip", strict=True, allowed=["under_budget"], scheduler=None,
             signals=[_sig("a", 6), _sig("b", 6)], script={"a": SKIPPED, "b": APPLIED}, states={}),
        dict(name="fatal_marker", strict=False, allowed=[], scheduler=None,
             signals=[_sig("a", 8), _sig("b", 8)],
             script={"a": APPLIED, "b": ("raise", "RuntimeError", "TRIATTN_FATAL_TRITON_SCORING_REQUIRED:score_failed:X")},
             states={}),
    ]


def run_scenario(execute_fn, signal_cls, result_cls, sc: dict, with_batch: bool = False) -> dict:
    executor = ScriptedExecutor(sc["script"], result_cls, with_batch=with_batch)
    store = RecordingStore(sc["states"])
    sched = None
    if sc["scheduler"] is not None:
        sched = types.SimpleNamespace(scheduled_cached_reqs=types.SimpleNamespace(**sc["scheduler"]))
    signals = {s["req_id"]: signal_cls(**s) for s in sc["signals"]}
    log = logging.getLogger("runner_action_scenarios")
    log.disabled = True
    raised, events = None, None
    try:
        events = execute_fn(executor=executor, state_store=store, scheduler_output=sched, signals=signals,
                            strict_no_downgrade=sc["strict"], allowed_strict_skip_reasons=set(sc["allowed"]),
                            logger=log, log_decisions=True)
    except Exception as exc:  # the driver's fatal errors are part of its contract
        raised = [type(exc).__name__, str(exc)]
    return {"events": events, "store_calls": store.calls, "raised": raised}
