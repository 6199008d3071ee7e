"""Scripted inputs for the scheduler-side pieces (trigger planner, effective-length tracker, allocation-sync
attributes, block-pool reclaim).  The fixture generator replays them on the reference's classes and functions, the
test on this package's; every returned value, every recorded pool call and every final state must agree."""
from __future__ import annotations

import dataclasses
import types

# ---------------------------------------------------------------------------------------------- trigger planner
PLANNER_CONFIGS = {
    "default": dict(kv_budget=2048, divide_length=128, protect_prefill=False, include_prefill_in_budget=False,
                    enable_kv_usage_trigger=False, kv_usage_trigger=0.98, kv_usage_release=0.90),
    "protected_prompt": dict(kv_budget=512, divide_length=64, protect_prefill=True, include_prefill_in_budget=False,
                             enable_kv_usage_trigger=False, kv_usage_trigger=0.98, kv_usage_release=0.90),
    "prompt_in_budget": dict(kv_budget=512, divide_length=64, protect_prefill=True, include_prefill_in_budget=True,
                             enable_kv_usage_trigger=False, kv_usage_trigger=0.98, kv_usage_release=0.90),
    "pool_pressure": dict(kv_budget=2048, divide_length=128, protect_prefill=False, include_prefill_in_budget=False,
                          enable_kv_usage_trigger=True, kv_usage_trigger=0.9, kv_usage_release=0.5),
}
PLANNER_CALLS = [
    dict(req_id="a", estimated_cache_len=2175, prefill_len=100, step=1),
    dict(req_id="a", estimated_cache_len=2176, prefill_len=100, step=2, scheduled_tokens=0),
    dict(req_id="b", estimated_cache_len=600, prefill_len=50, step=3, kv_usage=0.95, scheduled_tokens=7),
    dict(req_id="b", estimated_cache_len=575, prefill_len=-3, step=4, kv_usage=0.7),
    dict(req_id="b", estimated_cache_len=626, prefill_len=50, step=5, kv_usage=None),
    dict(req_id="c", estimated_cache_len=10, prefill_len=5, step=6, kv_usage=0.5),
    dict(req_id="c", estimated_cache_len=10, prefill_len=5, step=7, kv_usage=0.6),
    dict(req_id="c", estimated_cache_len=5000, prefill_len=4000, step=8, kv_usage=0.91),
]


def replay_planner(planner_cls) -> dict:
    out = {}
    for name, cfg in PLANNER_CONFIGS.items():
        planner = planner_cls(types.SimpleNamespace(**cfg))
        out[name] = [dataclasses.asdict(planner.build_signal(**kw)) for kw in PLANNER_CALLS]
    return out


# ---------------------------------------------------------------------------------------------- length tracker
TRACKER_CALLS = [
    ("observe_num_computed", ("a", 100)), ("observe_num_computed", ("a", 2177)),
    ("apply_compression", ("a", 2048, 2177)), ("observe_num_computed", ("a", 2178)),
    ("observe_num_computed", ("a", 2300)), ("observe_num_computed", ("a", 2200)),
    ("observe_num_computed", ("a", 10)), ("has_effective_len_override", ("a",)),
    ("has_effective_len_override", ("b",)), ("reset_request", ("a", 55)), ("observe_num_computed", ("a", 60)),
    ("apply_compression", ("b", -4, -9)), ("observe_num_computed", ("b", 3)), ("has_any_effective_len_overrides", ()),
    ("remove_request", ("b",)), ("remove_request", ("zz",)), ("has_any_effective_len_overrides", ()),
    ("observe_num_computed", ("c", -5)),
]


def replay_tracker(tracker) -> list:
    out = []
    for name, args in TRACKER_CALLS:
        ret = getattr(tracker, name)(*args)
        snap = {k: list(v) for k, v in sorted(tracker.snapshot().items())}
        out.append({"call": name, "returned": ret, "snapshot": snap})
    return out


# ---------------------------------------------------------------------------------------------- allocation sync
SYNC_CALLS = [
    ("update", dict(num_computed_tokens=3000), 2048), ("prepare", None, None), ("resolve", None, None),
    ("update", dict(num_computed_tokens=3001), 5000), ("prepare", None, None), ("resolve", None, None),
    ("update", dict(num_computed_tokens=4000), 1000), ("prepare", dict(num_computed_tokens=0), None),
    ("resolve", None, None), ("update", dict(num_computed_tokens=4000), 1000),
    ("prepare", dict(num_computed_tokens=2000), None), ("update", dict(num_computed_tokens="x"), 7),
    ("update", dict(num_computed_tokens=50), -3), ("prepare", None, None), ("resolve", None, None), ("clear", None, None),
    ("resolve", None, None),
]


def replay_allocation_sync(mod) -> list:
    """``mod`` offers the four functions and the two attribute names."""
    req = types.SimpleNamespace(num_computed_tokens=0)
    out = []
    for op, attrs, arg in SYNC_CALLS:
        for k, v in (attrs or {}).items():
            setattr(req, k, v)
        if op == "update":
            ret = mod.update_request_effective_kv_offset(request=req, cache_len_after=arg)
        elif op == "prepare":
            ret = mod.prepare_request_effective_num_computed(req)
        elif op == "resolve":
            ret = mod.resolve_request_effective_num_computed(req)
        else:
            ret = mod.clear_request_allocation_sync_state(req)
        out.append({"op": op, "returned": ret, "offset": getattr(req, mod.EFFECTIVE_KV_OFFSET_ATTR, "absent"),
                    "effective": getattr(req, mod.EFFECTIVE_NUM_COMPUTED_ATTR, "absent")})
    out.append({"op": "none", "returned": [mod.update_request_effective_kv_offset(request=None, cache_len_after=1),
                                            mod.prepare_request_effective_num_computed(None),
                                            mod.resolve_request_effective_num_computed(None)]})
    return out


# ---------------------------------------------------------------------------------------------- block-pool reclaim
class _Block:
    def __init__(self, block_id, hashed):
        self.block_id = block_id
        self.block_hash = ("h", block_id) if hashed else None


class _Pool:
    def __init__(self, log, gid, can_evict=True):
        self._log, self._gid = log, gid
        if can_evict:
            self._maybe_evict_cached_block = lambda block: log.append(["evict", gid, block.block_id])

    def free_blocks(self, blocks):
        self._log.append(["free", self._gid, [b.block_id for b in blocks]])


def _ev(req_id="a", after=2048, status="applied", **more):
    return dict(req_id=req_id, status=status, cache_len_after=after, step=3, **more)


def _grp(gid, after, before=None, **more):
    g = dict(gid=gid, block_ids_after=after, **more)
    if before is not None:
        g["block_ids_before"] = before
    return g


def _ids(lo, hi):
    return list(range(lo, hi))


# managers: per group {req_id: (first block id, number of blocks, ids of hashed blocks)}; cached: {req_id: n} per group
RECLAIM_CASES = [
    dict(name="explicit_payload_two_groups", block_size=16,
         managers=[{"a": (100, 137, {230, 236})}, {"a": (500, 137, set())}], cached=[{"a": 137}, {}],
         requests={"a": 2177},
         events=[_ev(block_reclaim={"groups": [_grp(0, _ids(100, 228), _ids(100, 237)), _grp(1, _ids(500, 628))]})]),
    dict(name="blocks_appended_after_the_hook", block_size=16, managers=[{"a": (0, 140, {139})}], cached=[{"a": 140}],
         requests={"a": 2200},
         events=[_ev(scheduled_tokens=40, block_reclaim={"groups": [_grp(0, _ids(0, 128), _ids(0, 137))]})]),
    dict(name="no_payload_single_token_step", block_size=16, managers=[{"a": (0, 137, {130})}, {"b": (900, 3, set())}],
         cached=[{"a": 130}, {}], requests={"a": 2177, "b": 40},
         events=[_ev(), _ev(req_id="b", after=40), _ev(req_id="ghost"), _ev(status="skipped"), _ev(after="2048"),
                 dict(status="applied", cache_len_after=5)]),
    dict(name="no_payload_during_prefill", block_size=16, managers=[{"a": (0, 137, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev(scheduled_tokens=64)]),
    dict(name="payload_misses_a_group", block_size=16, managers=[{"a": (0, 137, set())}, {"a": (300, 137, {436})}],
         cached=[{}, {"a": 137}], requests={"a": 2177},
         events=[_ev(block_reclaim={"groups": [_grp(0, _ids(0, 128)), "junk", _grp(7, [1]), _grp("0", [1]),
                                               _grp(1, "x"), _grp(1, [300, "301"])]})]),
    dict(name="payload_misses_a_group_during_prefill", block_size=16,
         managers=[{"a": (0, 137, set())}, {"a": (300, 137, set())}], cached=[{}, {}], requests={"a": 2177},
         events=[_ev(scheduled_tokens=9, block_reclaim={"groups": [_grp(0, _ids(0, 128))]})]),
    dict(name="reclaim_disabled", block_size=16, reclaim=False, managers=[{"a": (0, 137, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev()]),
    dict(name="zero_length_and_block_size_zero", block_size=0, managers=[{"a": (0, 5, {1})}], cached=[{"a": 9}],
         requests={"a": 5}, events=[_ev(after=0), _ev(after=-3)]),
    dict(name="pool_without_evict_and_no_pool", block_size=16, can_evict=False, no_pool_gids=[1],
         managers=[{"a": (0, 137, {131})}, {"a": (300, 137, set())}], cached=[{}, {}], requests={"a": 2177},
         events=[_ev()]),
    dict(name="error_prefix_mismatch", block_size=16, managers=[{"a": (0, 137, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev(block_reclaim={"groups": [_grp(0, _ids(1, 129))]})]),
    dict(name="error_duplicate_ids", block_size=16, managers=[{"a": (0, 137, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev(block_reclaim={"groups": [_grp(0, [0, 1, 1])]})]),
    dict(name="error_longer_than_held", block_size=16, managers=[{"a": (0, 4, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev(block_reclaim={"groups": [_grp(0, _ids(0, 9))]})]),
    dict(name="error_insufficient_shrink", block_size=16, managers=[{"a": (0, 137, set())}], cached=[{}],
         requests={"a": 2177}, events=[_ev(block_reclaim={"groups": [_grp(0, _ids(0, 130))]})]),
    dict(name="insufficient_shrink_tolerated", block_size=16, require=False, managers=[{"a": (0, 137, set())}],
         cached=[{}], requests={"a": 2177}, events=[_ev(block_reclaim={"groups": [_grp(0, _ids(0, 130))]})]),
    dict(name="managers_not_a_list", block_size=16, managers=None, cached=[], requests={"a": 2177},
         events=[_ev(), _ev(block_reclaim={"groups": [_grp(0, [1])]})]),
]


def run_reclaim_case(apply_fn, tracker_cls, case: dict) -> dict:
    """``apply_fn(scheduler_like, events)``; returns everything the call changed (or the error it raised)."""
    log = []
    managers = None
    if case["managers"] is not None:
        managers = []
        for gid, spec in enumerate(case["managers"]):
            pool = None if gid in case.get("no_pool_gids", []) else _Pool(log, gid, case.get("can_evict", True))
            managers.append(types.SimpleNamespace(
                req_to_blocks={r: [_Block(first + i, first + i in hashed) for i in range(n)]
                               for r, (first, n, hashed) in spec.items()},
                num_cached_block=dict(case["cached"][gid]), block_pool=pool))
    requests = {r: types.SimpleNamespace(num_computed_tokens=n) for r, n in case["requests"].items()}
    sched = types.SimpleNamespace(
        kv_cache_manager=types.SimpleNamespace(coordinator=types.SimpleNamespace(single_type_managers=managers)),
        block_size=case["block_size"], requests=requests, _effective_len_tracker=tracker_cls(),
        triattention_config=types.SimpleNamespace(enable_experimental_block_reclaim=case.get("reclaim", True),
                                                  require_physical_reclaim=case.get("require", True)))
    error = None
    try:
        apply_fn(sched, case["events"])
    except RuntimeError as exc:
        error = str(exc)
    return {
        "error": error, "pool_calls": log,
        "blocks": [{r: [b.block_id for b in bl] for r, bl in m.req_to_blocks.items()} for m in managers or []],
        "cached": [dict(m.num_cached_block) for m in managers or []],
        "tracker": {k: list(v) for k, v in sorted(sched._effective_len_tracker.snapshot().items())},
        "offsets": {r: getattr(q, "_triattention_effective_kv_offset", "absent") for r, q in requests.items()},
    }


# ---------------------------------------------------------------------------------------------- the scheduler's step
STEP_CONFIGS = {
    "length_trigger": dict(pool_blocks=100),
    "small_pool_caps_the_step": dict(pool_blocks=6),
    "pool_pressure_trigger": dict(pool_blocks=100, enable_kv_usage_trigger=True, kv_usage_trigger=0.9, kv_usage_release=0.5),
    "compression_disabled": dict(pool_blocks=100, disable_compression=True),
    "protected_prompt": dict(pool_blocks=100, protect_prefill=True),
}
_STEP_CFG_BASE = dict(kv_budget=64, divide_length=16, protect_prefill=False, include_prefill_in_budget=False,
                      enable_kv_usage_trigger=False, kv_usage_trigger=0.98, kv_usage_release=0.9, disable_compression=False,
                      enable_experimental_block_reclaim=True, require_physical_reclaim=True, log_decisions=False)

# per step: new requests (id, prompt tokens, computed so far), tokens scheduled, computed counters before the step,
# pool usage, what comes back from the worker (events on the runner's output, or on the scheduler output)
STEP_SCRIPT = [
    dict(new=[("a", 70, 0), ("b", 20, 0)], sched={"a": 40, "b": 20}, computed={"a": 0, "b": 0}, usage=0.2),
    dict(new=[("a", 70, 40)], sched={"a": 30, "b": 1, "ghost": 1}, computed={"a": 40, "b": 20}, usage=0.95),
    dict(sched={"a": 1, "b": 1}, computed={"a": 70, "b": 21}, usage=0.7),
    dict(sched={"a": 1, "b": 1}, computed={"a": 79, "b": 22}, usage=0.7,
         events_on="runner", events=[dict(status="applied", req_id="a", cache_len_after=64, step=4, scheduled_tokens=1,
                                          block_reclaim={"groups": [dict(gid=0, block_ids_after=[0, 1, 2, 3])]})]),
    dict(sched={"a": 1, "b": 1}, computed={"a": 80, "b": 23}, usage=0.4),
    dict(sched={"a": 1, "b": 1}, computed={"a": 95, "b": 24}, usage=0.4, finished=["b"],
         events_on="scheduler", events=[dict(status="applied", req_id="a", cache_len_after=64, step=6, scheduled_tokens=1),
                                        dict(status="skipped", req_id="b", cache_len_after=None, step=6)]),
    dict(sched={"a": 1, "c": 1}, computed={"a": 96, "c": 300}, usage=0.4, resumed=["c"], prompt={"c": 250}),
    dict(sched={"a": 1}, computed={"a": 97}, usage=0.4, finished=["a", "c"]),
]


def run_scheduler_steps(api, cfg_over: dict) -> list:
    """``api.attach(scheduler, cfg)``, ``api.schedule(scheduler, base_schedule)``,
    ``api.update(scheduler, scheduler_output, model_runner_output, base_update)``."""
    over = dict(cfg_over)
    pool_blocks = over.pop("pool_blocks")
    cfg = types.SimpleNamespace(**{**_STEP_CFG_BASE, **over})
    log = []
    pool = _Pool(log, 0)
    pool.num_gpu_blocks = pool_blocks
    manager = types.SimpleNamespace(req_to_blocks={"a": [_Block(i, False) for i in range(6)]}, num_cached_block={},
                                    block_pool=pool)
    kvm = types.SimpleNamespace(usage=0.0, block_pool=pool,
                                coordinator=types.SimpleNamespace(single_type_managers=[manager]))
    sched = types.SimpleNamespace(requests={}, kv_cache_manager=kvm, running=[], block_size=16,
                                  max_num_scheduled_tokens=8192)
    api.attach(sched, cfg)
    caps = []
    out = []
    for st in STEP_SCRIPT:
        for r, n in st["computed"].items():
            if r in sched.requests:
                sched.requests[r].num_computed_tokens = n
            else:
                sched.requests[r] = types.SimpleNamespace(num_computed_tokens=n, num_prompt_tokens=st.get("prompt", {}).get(r, 0))
        for r, prompt, _done in st.get("new", []):
            sched.requests[r].num_prompt_tokens = prompt
        sched.running = list(sched.requests.values())
        kvm.usage = st["usage"]
        so = types.SimpleNamespace(
            num_scheduled_tokens=dict(st["sched"]), finished_req_ids=list(st.get("finished", [])),
            scheduled_new_reqs=[types.SimpleNamespace(req_id=r, num_computed_tokens=done, prompt_token_ids=[0] * prompt)
                                for r, prompt, done in st.get("new", [])],
            scheduled_cached_reqs=types.SimpleNamespace(req_ids=[r for r in st["sched"] if r in sched.requests],
                                                        resumed_req_ids=list(st.get("resumed", []))))

        def base_schedule(s, _so=so):
            caps.append(s.max_num_scheduled_tokens)
            return _so

        got = api.schedule(sched, base_schedule)
        rec = {"step": got.triattention_step, "cap_seen": caps[-1], "cap_after": sched.max_num_scheduled_tokens,
               "signals": {k: dataclasses.asdict(v) for k, v in got.triattention_signals.items()},
               "effective_markers": {r: getattr(q, "_triattention_effective_num_computed_tokens", "absent")
                                     for r, q in sched.requests.items()}}
        mro = types.SimpleNamespace()
        if st.get("events_on") == "runner":
            mro.triattention_compression_events = st["events"]
        elif st.get("events_on") == "scheduler":
            so.triattention_compression_events = st["events"]
        stats = types.SimpleNamespace(kv_cache_usage=-1.0)
        outputs = api.update(sched, so, mro, lambda s, a, b, _stats=stats: {0: types.SimpleNamespace(scheduler_stats=_stats),
                                                                             1: types.SimpleNamespace()})
        rec.update({
            "usage_in_stats": outputs[0].scheduler_stats.kv_cache_usage,
            "blocks": {r: [b.block_id for b in bl] for r, bl in manager.req_to_blocks.items()},
            "pool_calls": list(log),
            "tracker": {k: list(v) for k, v in sorted(sched._effective_len_tracker.snapshot().items())},
            "prefill_lens": dict(sched._prefill_lens), "thresholds": dict(sched._length_threshold_cache),
            "offsets": {r: getattr(q, "_triattention_effective_kv_offset", "absent") for r, q in sched.requests.items()},
        })
        for r in st.get("finished", []):
            sched.requests.pop(r, None)
        out.append(rec)
    return out


# ---------------------------------------------------------------------------------------------- slot allocation
ALLOC_CASES = [
    dict(name="no_reclaim", computed=500, attrs={}),
    dict(name="offset_applied", computed=500, attrs={"_triattention_effective_kv_offset": 120}, kwargs={"x": 1}),
    dict(name="offset_larger_than_progress", computed=100, attrs={"_triattention_effective_kv_offset": 120}),
    dict(name="progress_zero", computed=0, attrs={"_triattention_effective_kv_offset": 120}),
    dict(name="non_integer_progress", computed="12", attrs={"_triattention_effective_kv_offset": 5}),
    dict(name="base_raises", computed=500, attrs={"_triattention_effective_kv_offset": 120}, raises=True),
    dict(name="stale_marker_without_offset", computed=500, attrs={"_triattention_effective_num_computed_tokens": 300}),
]


def run_alloc_case(fn, case) -> dict:
    """``fn(manager, request, num_new_tokens, *args, base_allocate, **kwargs)``"""
    req = types.SimpleNamespace(num_computed_tokens=case["computed"], **case["attrs"])
    seen = {}

    def base(manager, request, num_new_tokens, *args, **kwargs):
        seen.update(computed=request.num_computed_tokens, num_new=num_new_tokens, args=list(args), kwargs=dict(kwargs))
        if case.get("raises"):
            raise ValueError("pool exhausted")
        return "blocks"

    out = {"error": None, "returned": None}
    try:
        out["returned"] = fn("mgr", req, 7, "extra", base_allocate=base, **case.get("kwargs", {}))
    except ValueError as exc:
        out["error"] = str(exc)
    out["seen"] = seen
    out["computed_after"] = req.num_computed_tokens
    out["marker_after"] = getattr(req, "_triattention_effective_num_computed_tokens", "absent")
    return out


def run_boundary_predicates(has_boundary, queue_pending, signal_cls) -> dict:
    def sig(should):
        return signal_cls(req_id="a", should_compress=should, reason="none", estimated_cache_len=1, step=1, kv_usage=None,
                          protect_prefill=False, prefill_len=0, scheduled_tokens=1)

    so = types.SimpleNamespace
    marked, plain = so(_triattention_force_boundary_sync=True), so()
    return {
        "boundary": [has_boundary(so()), has_boundary(so(triattention_signals={})),
                     has_boundary(so(triattention_signals={"a": sig(False)})),
                     has_boundary(so(triattention_signals={"a": sig(False), "b": sig(True)})),
                     has_boundary(so(triattention_signals=[sig(True)]))],
        "queue": [queue_pending(None), queue_pending([]), queue_pending([("f", plain, "e")]),
                  queue_pending([("f", plain), ("f", marked, "e")]), queue_pending([("f",), "junk", (1, marked)]),
                  queue_pending(5)],
    }
