"""Four scheduler outputs in a row for the worker's step life cycle (new / finished / preempted / resumed requests,
signals, actions): replayed on the reference's modules by the fixture generator and on this package's by the test."""
from __future__ import annotations

import dataclasses
import logging
import types


def _sig(req_id, step, est, should=False, sched=1, prefill=100, protect=False):
    return dict(req_id=req_id, should_compress=should, reason="length_threshold" if should else "none",
                estimated_cache_len=est, step=step, kv_usage=None, protect_prefill=protect, prefill_len=prefill,
                scheduled_tokens=sched)


STEPS = [
    dict(new=[dict(req_id="a", prompt_token_ids=list(range(100))), dict(req_id="b", num_prompt_tokens="3000", prompt_token_ids_len=2900),
              dict(req_id="c", prefill_token_ids=[1, 2, 3])],
         finished=[], preempted=None, cached=None, step=1,
         signals=[_sig("a", 1, 2177, should=True), _sig("b", 1, 3001, prefill=3000, protect=True)],
         script={"a": {"applied": True, "reason": "kv_compacted:per_head", "cache_len_after": 2048}}),
    dict(new=[], finished=[], preempted=["b"], cached=dict(req_ids=["a"], num_computed_tokens=[2177]), step=2,
         signals=[_sig("a", 2, 9999, should=True), _sig("c", 2, 4, prefill=3)], script={}),
    dict(new=[], finished=["c"], preempted=[], cached=dict(req_ids=["a", "b"], resumed_req_ids=["b"], num_computed_tokens=[2178, 3001]),
         step=None, signals=[_sig("a", 3, 1, sched=5), _sig("b", 3, 3002, should=True, prefill=3000, protect=True)],
         script={"b": {"applied": False, "reason": "prefill_exceeds_budget"}}),
    dict(new=[], finished=["zz"], preempted=None, cached=dict(req_ids=["a"], num_computed_tokens=[2300]), step=9,
         signals=[_sig("a", 9, 50, should=True, sched=1)],
         script={"a": {"applied": True, "reason": "kv_compacted:per_head", "cache_len_after": 2048}}),
]


class _Executor:
    def __init__(self, script, result_cls):
        self._script, self._cls = script, result_cls

    def execute(self, req_id, signal, scheduler_output):
        d = dict(self._script[req_id])
        return self._cls(applied=bool(d.get("applied")), reason=str(d.get("reason")), cache_len_after=d.get("cache_len_after"),
                         details=d)


def replay(mod, store, signal_cls, result_cls) -> list:
    """``mod`` offers the life-cycle functions and execute_runner_compression_actions."""
    log = logging.getLogger("step_lifecycle")
    log.disabled = True
    out, last = [], 0
    for st in STEPS:
        so = types.SimpleNamespace(
            scheduled_new_reqs=[types.SimpleNamespace(**r) for r in st["new"]], finished_req_ids=list(st["finished"]),
            triattention_signals={s["req_id"]: signal_cls(**s) for s in st["signals"]})
        if st["preempted"] is not None:
            so.preempted_req_ids = list(st["preempted"])
        if st["cached"] is not None:
            so.scheduled_cached_reqs = types.SimpleNamespace(**st["cached"])
        if st["step"] is not None:
            so.triattention_step = st["step"]
        mod.register_new_requests(state_store=store, scheduler_output=so, protect_prefill=False)
        mod.cleanup_finished_requests(state_store=store, scheduler_output=so)
        mod.mark_preemptions(state_store=store, scheduler_output=so)
        mod.mark_resumed(state_store=store, scheduler_output=so)
        last, signals = mod.consume_runner_signals(state_store=store, scheduler_output=so, last_step=last, logger=log,
                                                   log_decisions=True)
        events = mod.execute_runner_compression_actions(
            executor=_Executor(st["script"], result_cls), state_store=store, scheduler_output=so, signals=signals,
            strict_no_downgrade=False, allowed_strict_skip_reasons=set(), logger=log, log_decisions=False)
        out.append({"step": last, "events": events,
                    "states": {k: dataclasses.asdict(v) for k, v in sorted(store.snapshot().items())}})
    return out
