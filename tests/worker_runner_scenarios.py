"""Scripted inputs for the worker's runner proxy: self-triggers, trimming of stale new block ids, the overrides of a
step, event attachment, and whole execute_model / sample_tokens steps.  The fixture generator replays them on the
reference's runner (methods called unbound on a stand-in where they need no engine), the test on this package's."""
from __future__ import annotations

import dataclasses
import logging
import types

import numpy as np

_LOG = logging.getLogger("worker_runner_scenarios")
_LOG.disabled = True

BASE_CFG = dict(kv_budget=64, divide_length=16, protect_prefill=False, include_prefill_in_budget=False,
                enable_experimental_kv_compaction=True, log_decisions=False)


def _cfg(**over):
    return types.SimpleNamespace(**{**BASE_CFG, **over})


def _sig(signal_cls, req_id, est, should=True, sched=1, step=5, prefill=10):
    return signal_cls(req_id=req_id, should_compress=should, reason="length_threshold" if should else "none",
                      estimated_cache_len=est, step=step, kv_usage=None, protect_prefill=False, prefill_len=prefill,
                      scheduled_tokens=sched)


def _store(store_cls, spec):
    """spec: {req_id: (prefill_len, cache_len, compressed_to or None)}"""
    store = store_cls()
    for req_id, (prefill, cache_len, compressed_to) in spec.items():
        store.ensure(req_id=req_id, prefill_len=prefill, protect_prefill=False)
        store.update_cache_len(req_id, cache_len, step=1)
        if compressed_to is not None:
            store.mark_compressed(req_id, step=1, cache_len=compressed_to, scheduled_tokens=1, scheduler_nct=cache_len)
    return store


def _runner(rows=None, blocks_per_row=None, block_size=16, requests=None, capacity=None, nested=True):
    """Stand-in base runner: ``rows`` {req_id: row}, ``blocks_per_row`` list, ``requests`` {req_id: computed tokens}."""
    r = types.SimpleNamespace()
    if requests is not None:
        r.requests = {k: types.SimpleNamespace(num_computed_tokens=v) for k, v in requests.items()}
    if rows is not None:
        inner = types.SimpleNamespace(num_blocks_per_row=np.asarray(blocks_per_row, dtype=np.int32))
        table = types.SimpleNamespace(block_tables=[inner]) if nested else inner
        if capacity is not None:
            table.max_num_blocks_per_req = capacity
        r.input_batch = types.SimpleNamespace(req_id_to_index=dict(rows), block_table=table)
        r.cache_config = types.SimpleNamespace(block_size=block_size)
    return r


# ---------------------------------------------------------------------------------------------- self-triggers
def self_trigger_cases(signal_cls):
    return [
        dict(name="compressed_request_by_its_own_count", cfg=_cfg(), store={"a": (10, 200, 79)},
             runner=_runner(), sched={"a": 1}, signals={}),
        dict(name="decode_trigger_of_the_scheduler_stands", cfg=_cfg(), store={"a": (10, 200, 79)},
             runner=_runner(), sched={"a": 1}, signals={"a": _sig(signal_cls, "a", 999)}),
        dict(name="prefill_trigger_corrected_from_block_table", cfg=_cfg(), store={"a": (10, 40, None)},
             runner=_runner(rows={"a": 2}, blocks_per_row=[0, 0, 6]), sched={"a": 8},
             signals={"a": _sig(signal_cls, "a", 48, sched=8)}),
        dict(name="block_table_flat_and_below_threshold", cfg=_cfg(), store={"a": (10, 40, None)},
             runner=_runner(rows={"a": 0}, blocks_per_row=[4], nested=False), sched={"a": 1}, signals={}),
        dict(name="runner_counter_fallback", cfg=_cfg(), store={"a": (10, 40, None), "b": (10, 40, None)},
             runner=_runner(requests={"a": 79, "b": 78}), sched={"a": 1, "b": 1}, signals={}),
        dict(name="no_state_or_no_request", cfg=_cfg(), store={"b": (10, 40, None)}, runner=_runner(requests={"a": 500}),
             sched={"a": 1, "b": 1}, signals={}),
        dict(name="protected_prompt_raises_the_threshold", cfg=_cfg(protect_prefill=True),
             store={"a": (30, 200, 100), "b": (30, 200, 110)}, runner=_runner(), sched={"a": 1, "b": 1}, signals={}),
        dict(name="unscheduled_non_trigger_signal_replaced", cfg=_cfg(), store={"a": (10, 200, 90)}, runner=_runner(),
             sched={"a": 0}, signals={"a": _sig(signal_cls, "a", 70, should=False)}),
        dict(name="compaction_switched_off", cfg=_cfg(enable_experimental_kv_compaction=False),
             store={"a": (10, 200, 90)}, runner=_runner(), sched={"a": 1}, signals={}),
        dict(name="zero_block_size", cfg=_cfg(), store={"a": (10, 40, None)},
             runner=_runner(rows={"a": 0}, blocks_per_row=[9], block_size=0, requests={"a": 100}), sched={"a": 1},
             signals={}),
    ]


def run_self_trigger(fn, store_cls, case) -> dict:
    """``fn(base_runner, config, store, scheduler_output, signals, last_step) -> signals``"""
    so = types.SimpleNamespace(num_scheduled_tokens=dict(case["sched"]))
    out = fn(case["runner"], case["cfg"], _store(store_cls, case["store"]), so, dict(case["signals"]), 7)
    return {k: dataclasses.asdict(v) for k, v in out.items()}


# ---------------------------------------------------------------------------------------------- stale new block ids
TRIM_CASES = [
    dict(name="trimmed_to_the_room_left", store={"a": (10, 200, 64), "b": (10, 50, None)},
         runner=dict(rows={"a": 0, "b": 1}, blocks_per_row=[6, 2], capacity=8), req_ids=["a", "b"],
         new_block_ids=[([1, 2, 3, 4], [5, 6, 7]), ([9, 9, 9, 9, 9, 9, 9], )]),
    dict(name="fits", store={"a": (10, 200, 64)}, runner=dict(rows={"a": 0}, blocks_per_row=[6], capacity=8),
         req_ids=["a"], new_block_ids=[([1, 2], )]),
    dict(name="row_already_full", store={"a": (10, 200, 64)}, runner=dict(rows={"a": 0}, blocks_per_row=[9], capacity=8),
         req_ids=["a"], new_block_ids=[[[1], "x"]]),
    dict(name="none_and_unknown_rows", store={"a": (10, 200, 64), "c": (10, 200, 64)},
         runner=dict(rows={"a": 0}, blocks_per_row=[7], capacity=8), req_ids=["a", "c", "zz"],
         new_block_ids=[None, ([1, 2, 3], ), ([1, 2, 3], )]),
    dict(name="length_mismatch", store={"a": (10, 200, 64)}, runner=dict(rows={"a": 0}, blocks_per_row=[7], capacity=8),
         req_ids=["a"], new_block_ids=[([1, 2], ), ([3], )]),
    dict(name="no_capacity_attribute", store={"a": (10, 200, 64)}, runner=dict(rows={"a": 0}, blocks_per_row=[7]),
         req_ids=["a"], new_block_ids=[([1, 2, 3], )]),
]


def run_trim(fn, store_cls, case) -> list:
    """``fn(base_runner, store, scheduler_output)``; returns the new-block-id lists afterwards."""
    so = types.SimpleNamespace(scheduled_cached_reqs=types.SimpleNamespace(
        req_ids=list(case["req_ids"]), new_block_ids=list(case["new_block_ids"])))
    fn(_runner(**case["runner"]), _store(store_cls, case["store"]), so)
    return [None if g is None else [list(x) if isinstance(x, (list, tuple)) else x for x in g]
            for g in so.scheduled_cached_reqs.new_block_ids]


# ---------------------------------------------------------------------------------------------- overrides of a step
OVERRIDE_CASES = [
    dict(name="one_compressed_of_three", store={"a": (10, 200, 64), "b": (10, 50, None), "c": (10, 90, None)},
         runner=dict(rows={"a": 2, "b": 0, "c": 1}, blocks_per_row=[4, 6, 5], requests={"a": 201, "b": 50, "c": 90}),
         sched={"b": 1, "a": 1, "c": 3}, cached=dict(req_ids=["a", "b", "c"], num_computed_tokens=[201, 50, 90])),
    dict(name="two_compressed", store={"a": (10, 200, 64), "b": (10, 300, 64)},
         runner=dict(rows={"a": 0, "b": 1}, blocks_per_row=[5, 5], requests={"a": 203, "b": 301}),
         sched={"a": 1, "b": 2}, cached=dict(req_ids=["a", "b"], num_computed_tokens=[203, 301])),
    dict(name="nothing_compressed", store={"a": (10, 50, None)},
         runner=dict(rows={"a": 0}, blocks_per_row=[4], requests={"a": 50}), sched={"a": 1},
         cached=dict(req_ids=["a"], num_computed_tokens=[50])),
    dict(name="no_row_lookup", store={"a": (10, 200, 64)}, runner=dict(requests={"a": 201}), sched={"a": 1},
         cached=dict(req_ids=["a"], num_computed_tokens=[201])),
]


def run_overrides(prepare_fn, needs_fn, store_cls, case) -> dict:
    store = _store(store_cls, case["store"])
    so = types.SimpleNamespace(num_scheduled_tokens=dict(case["sched"]), triattention_step=2,
                               scheduled_cached_reqs=types.SimpleNamespace(**case["cached"]))
    runner = _runner(**case["runner"])
    ov = prepare_fn(base_runner=runner, state_store=store, scheduler_output=so)
    d = {k: getattr(ov, k) for k in ("seq_base_map", "pos_delta_map", "single_seq_base", "single_pos_delta",
                                      "expected_req_row_indices", "expected_query_lens")}
    d = {k: ({str(a): b for a, b in v.items()} if isinstance(v, dict) else (list(v) if isinstance(v, tuple) else v))
         for k, v in d.items()}
    d["needs"] = needs_fn(store, so)
    d["needs_nothing_scheduled"] = needs_fn(store, types.SimpleNamespace(num_scheduled_tokens={}))
    only_any = types.SimpleNamespace(has_active_compressed_requests=store.has_active_compressed_requests)
    d["needs_with_a_plain_store"] = needs_fn(only_any, so)
    d["needs_with_no_checker"] = needs_fn(types.SimpleNamespace(), so)
    return d


# ---------------------------------------------------------------------------------------------- events on outputs
class _Sealed:
    __slots__ = ()


def run_attach(mod) -> dict:
    ev = [{"status": "applied", "req_id": "a"}, {"status": "skipped", "req_id": "b"}]
    out = {}
    o = types.SimpleNamespace()
    r, left = mod.attach_execute_model_compression_events(output=o, pending_events=list(ev), scheduler_output=None)
    out["on_output"] = [getattr(r, "triattention_compression_events", "absent"), left]
    so = types.SimpleNamespace()
    r, left = mod.attach_execute_model_compression_events(output=None, pending_events=list(ev), scheduler_output=so)
    out["on_scheduler_output"] = [r, getattr(so, "triattention_compression_events", "absent"), left]
    so = types.SimpleNamespace()
    r, left = mod.attach_execute_model_compression_events(output=None, pending_events=[], scheduler_output=so)
    out["nothing_pending"] = [r, getattr(so, "triattention_compression_events", "absent"), left]
    r, left = mod.attach_execute_model_compression_events(output=None, pending_events=list(ev), scheduler_output=None)
    out["nowhere_to_go"] = [r, left]
    r, left = mod.attach_execute_model_compression_events(output=_Sealed(), pending_events=list(ev))
    out["sealed_output"] = [type(r).__name__, left]
    o = types.SimpleNamespace()
    r, left = mod.attach_sample_tokens_compression_events(output=o, pending_events=list(ev))
    out["sample_tokens"] = [getattr(r, "triattention_compression_events", "absent"), left]
    r, left = mod.attach_sample_tokens_compression_events(output=None, pending_events=list(ev))
    out["sample_tokens_none"] = [r, left]
    return out


# ---------------------------------------------------------------------------------------------- whole steps
def run_steps(runner_cls, config_obj, signal_cls) -> list:
    """Eight steps of three requests through ``execute_model`` / ``sample_tokens`` of the proxy on a runner without batch
    structures (no row lookup: no overrides, no block-table work), with a scripted hook."""
    calls = []
    base = types.SimpleNamespace(requests={})

    def hook(req_id, signal, scheduler_output):
        calls.append(["hook", req_id, signal.estimated_cache_len, signal.scheduled_tokens])
        if req_id == "b":
            return {"applied": False, "reason": "under_budget"}
        return {"applied": True, "reason": "kv_compacted:per_head", "cache_len_after": 64,
                "block_reclaim": {"mode": "truncate_tail", "groups": [{"gid": 0, "block_ids_after": [1, 2, 3, 4]}]}}

    def execute_model(scheduler_output, intermediate_tensors=None):
        calls.append(["execute_model", getattr(scheduler_output, "triattention_step", None), intermediate_tensors])
        return None if getattr(scheduler_output, "async_mode", False) else types.SimpleNamespace(tag="out")

    base.triattention_apply_compression = hook
    base.execute_model = execute_model
    base.sample_tokens = lambda grammar_output: types.SimpleNamespace(tag="sampled", grammar=grammar_output)
    base.some_engine_attribute = 42
    proxy = runner_cls(base, config_obj)
    out = [{"passthrough": proxy.some_engine_attribute,
            "store_on_runner": getattr(base, "_triattention_state_store", None) is proxy.state_store}]
    plan = [
        dict(step=1, new=[("a", 70), ("b", 20)], sched={"a": 70, "b": 20}, signals=[("a", 70, False, 70), ("b", 20, False, 20)]),
        dict(step=2, sched={"a": 1, "b": 1}, signals=[("a", 71, False, 1), ("b", 21, False, 1)], computed={"a": 70, "b": 20}),
        dict(step=3, sched={"a": 1, "b": 1}, signals=[("a", 80, True, 1), ("b", 90, True, 1)], computed={"a": 79, "b": 21}),
        dict(step=4, sched={"a": 1}, signals=[("a", 81, False, 1)], computed={"a": 80, "b": 22}, async_mode=True,
             sample=True),
        dict(step=5, sched={"a": 1, "b": 1}, signals=[], computed={"a": 94, "b": 23}, preempted=["b"]),
        dict(step=6, sched={"a": 1}, signals=[("a", 70, False, 1)], computed={"a": 95}, finished=["b"], async_mode=True,
             sample=True),
        # a trigger in asynchronous mode: the events travel on the scheduler output
        dict(step=7, new=[("c", 100)], sched={"a": 1, "c": 100}, signals=[("a", 95, True, 1), ("c", 100, False, 100)],
             computed={"a": 96}, async_mode=True, sample=True),
        # the scheduler says nothing about c, the worker triggers it itself (100 computed + 1 scheduled >= 80)
        dict(step=8, sched={"a": 1, "c": 1}, signals=[("a", 70, False, 1)], computed={"a": 97, "c": 100}),
    ]
    for st in plan:
        for r, n in (st.get("computed") or {}).items():
            base.requests[r] = types.SimpleNamespace(num_computed_tokens=n)
        so = types.SimpleNamespace(
            triattention_step=st["step"], num_scheduled_tokens=dict(st["sched"]),
            scheduled_new_reqs=[types.SimpleNamespace(req_id=r, prompt_token_ids=[0] * n) for r, n in st.get("new", [])],
            finished_req_ids=list(st.get("finished", [])), preempted_req_ids=list(st.get("preempted", [])),
            triattention_signals={r: _sig(signal_cls, r, est, should=should, sched=sched, step=st["step"], prefill=0)
                                  for r, est, should, sched in st["signals"]},
            async_mode=st.get("async_mode", False))
        result = proxy.execute_model(so, intermediate_tensors="it")
        rec = {"step": st["step"], "output": None if result is None else result.tag,
               "events_on_output": getattr(result, "triattention_compression_events", "absent") if result is not None else "absent",
               "events_on_scheduler_output": getattr(so, "triattention_compression_events", "absent")}
        if st.get("sample"):
            sampled = proxy.sample_tokens("g")
            rec["sampled"] = [sampled.tag, sampled.grammar, sampled.triattention_compression_events]
        rec["states"] = {k: dataclasses.asdict(v) for k, v in sorted(proxy.snapshot_states().items())}
        rec["calls"] = list(calls)
        calls.clear()
        out.append(rec)
    return out
