"""Scripted steps for the effective-length override builder: the fixture generator runs the reference's
``build_effective_sparse_overrides`` on them, the test runs this package's."""
from __future__ import annotations

import types


class _Key:
    """A scheduler key that is an object carrying the request id (newer engines)."""

    def __init__(self, request_id):
        self.request_id = request_id

    def __hash__(self):
        return hash(("key", self.request_id))

    def __eq__(self, other):
        return isinstance(other, _Key) and other.request_id == self.request_id


class _Store:
    def __init__(self, states: dict, any_compressed):
        self._states = {k: types.SimpleNamespace(**v) for k, v in states.items()}
        self._any = any_compressed

    def get(self, req_id):
        return self._states.get(req_id)

    def has_active_compressed_requests(self):
        if self._any == "raise":
            raise RuntimeError("x")
        return self._any


def _state(count=1, cur=2100, sem="estimated_with_scheduled", step=-1, prefill=100, nct=None, after=None):
    return dict(compression_count=count, current_cache_len=cur, current_cache_len_semantics=sem,
                current_cache_len_step=step, prefill_len=prefill, nct_at_last_compression=nct,
                cache_len_after_last_compression=after)


def scenarios() -> list:
    return [
        dict(name="nothing_compressed", any=False, states={}, index={"a": 0}, requests={"a": 500}, sched={"a": 1}),
        dict(name="stable_anchor_two_requests", any=True,
             states={"a": _state(nct=2175, after=2048), "b": _state(nct=9000, after=2048), "c": _state(count=0)},
             index={"a": 3, "b": 0, "c": 1}, requests={"a": 0, "b": 0, "c": 700},
             sched={"a": 1, "b": 1, "c": 1}, cached={"req_ids": ["a", "b", "c"], "num_computed_tokens": [2200, 9500, 700]}),
        dict(name="stable_anchor_single", any=True, states={"a": _state(nct=2175, after=2048)}, index={"a": 5},
             requests={"a": 0}, sched={"a": 1}, cached={"req_ids": ["a"], "num_computed_tokens": [2300]}),
        dict(name="fallback_estimated", any=True, states={"a": _state(cur=2100)}, index={"a": 2}, requests={"a": 2226},
             sched={"a": 1}),
        dict(name="fallback_pre_step_marker_match", any=True, states={"a": _state(cur=2100, sem="effective_pre_step", step=7)},
             index={"a": 2}, requests={"a": 2226}, sched={"a": 1}, step=7),
        dict(name="fallback_pre_step_marker_stale", any=True, states={"a": _state(cur=2100, sem="effective_pre_step", step=6)},
             index={"a": 2}, requests={"a": 2226}, sched={"a": 4}, step=7),
        dict(name="semantics_missing_raises", any=True, states={"a": _state(cur=2100, sem=None)}, index={"a": 2},
             requests={"a": 2226}, sched={"a": 1}),
        dict(name="events_without_compressed_state_raise", any=False, states={}, index={"a": 0}, requests={"a": 5},
             sched={"a": 1}, events=[{"status": "applied", "req_id": "a"}, {"status": "skipped", "req_id": "b"}]),
        dict(name="zero_delta_and_unknown_rows", any=True,
             states={"a": _state(cur=301), "b": _state(cur=900)}, index={"a": 0}, requests={"a": 300, "b": 100},
             sched={"a": 1, "b": 1, "zz": "many"}),
        dict(name="object_keys_and_checker_failure", any="raise", states={"a": _state(cur=2100)}, index={"a": 1},
             requests={"a": 4000}, sched_obj={"a": 1}),
        dict(name="chunked_prefill_lag", any=True,
             states={"a": _state(cur=2048, sem="effective_pre_step", step=3, prefill=3000)}, index={"a": 0},
             requests={"a": 2048}, sched={"a": 1}, step=3),
        dict(name="rows_from_input_batch_list", any=True, states={"a": _state(cur=2100)}, index=None, batch_ids=[None, "x", "a"],
             requests={"a": 2226}, sched={"a": 1}),
        dict(name="no_requests_dict", any=True, states={}, index={"a": 0}, requests=None, sched={"a": 1}),
        dict(name="nothing_scheduled", any=True, states={"a": _state()}, index={"a": 0}, requests={"a": 5}, sched={}),
    ]


def build_inputs(sc: dict):
    runner = types.SimpleNamespace()
    if sc.get("requests") is not None:
        runner.requests = {r: types.SimpleNamespace(num_computed_tokens=n) for r, n in sc["requests"].items()}
    if sc.get("index") is not None:
        runner.req_states = types.SimpleNamespace(req_id_to_index=dict(sc["index"]))
    if sc.get("batch_ids") is not None:
        runner.input_batch = types.SimpleNamespace(req_ids=lambda: list(sc["batch_ids"]))
    so = types.SimpleNamespace()
    if "sched_obj" in sc:
        so.num_scheduled_tokens = {_Key(r): n for r, n in sc["sched_obj"].items()}
    else:
        so.num_scheduled_tokens = dict(sc["sched"])
    if "cached" in sc:
        so.scheduled_cached_reqs = types.SimpleNamespace(**sc["cached"])
    if "step" in sc:
        so.triattention_step = sc["step"]
    return runner, _Store(sc["states"], sc["any"]), so


def run_scenario(build_fn, sc: dict) -> dict:
    runner, store, so = build_inputs(sc)
    try:
        seq, pos, one_seq, one_pos = build_fn(base_runner=runner, state_store=store, scheduler_output=so,
                                              compression_events=sc.get("events"))
    except Exception as exc:
        return {"raised": [type(exc).__name__, str(exc)]}
    as_pairs = lambda d: None if d is None else sorted([int(k), int(v)] for k, v in d.items())
    return {"raised": None, "seq_bases": as_pairs(seq), "pos_deltas": as_pairs(pos), "single_seq_base": one_seq,
            "single_pos_delta": one_pos}
