"""The worker-side action driver against the reference's own outputs (tests/golden/runner_action_cases.json,
produced by running runtime/runner_compression_actions.py:11-237 on the scripted scenarios)."""
from __future__ import annotations

import json
from pathlib import Path

import pytest

import runner_action_scenarios as ras
from triattention_b200 import runner_actions
from triattention_b200.constants import TRITON_SCORING_REQUIRED_MARKER
from triattention_b200.signals import CompressionSignal

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "runner_action_cases.json").read_text())


def _run(sc, with_batch=False):
    out = ras.run_scenario(runner_actions.execute_runner_compression_actions, CompressionSignal,
                           runner_actions.CompressionExecutionResult, sc, with_batch=with_batch)
    return json.loads(json.dumps(out))  # tuples -> lists, as in the stored fixture


@pytest.mark.parametrize("sc", ras.scenarios(), ids=lambda sc: sc["name"])
def test_per_request_execution_reproduces_the_reference(sc):
    """Executor without a batch entry: events, state-store calls (in order) and fatal errors are the reference's."""
    assert _run(sc) == GOLDEN[sc["name"]]


@pytest.mark.parametrize("sc", [s for s in ras.scenarios() if not any(isinstance(v, tuple) for v in s["script"].values())],
                         ids=lambda sc: sc["name"])
def test_batched_execution_gives_the_same_events(sc):
    """With an executor that runs the step's requests in one call nothing the scheduler sees changes."""
    assert _run(sc, with_batch=True) == GOLDEN[sc["name"]]


def test_a_failing_batch_reports_every_request():
    """One native call carries the whole step: if it raises, every request of the step gets the error event; in
    strict mode, or for the fatal marker, the error propagates as in the per-request loop."""
    by_name = {s["name"]: s for s in ras.scenarios()}
    soft = _run(by_name["soft_exception"], with_batch=True)
    assert soft["raised"] is None
    assert [(e["req_id"], e["status"], e["reason"]) for e in soft["events"]] == [
        ("a", "error", "executor_exception:ValueError"), ("b", "error", "executor_exception:ValueError")]
    assert [c[0] for c in soft["store_calls"]] == ["mark_compression_skipped"] * 2
    strict = _run(by_name["strict_exception"], with_batch=True)
    assert strict["raised"][0] == "RuntimeError" and TRITON_SCORING_REQUIRED_MARKER in strict["raised"][1]
    assert "executor_exception" in strict["raised"][1] and strict["store_calls"] == []
    fatal = _run(by_name["fatal_marker"], with_batch=True)
    assert fatal["raised"] == ["RuntimeError", "TRIATTN_FATAL_TRITON_SCORING_REQUIRED:score_failed:X"]


def test_runner_hook_executor_uses_the_batch_hook_when_present():
    import types
    calls = []

    def hook(req_id, signal, scheduler_output):
        calls.append(("one", req_id))
        return {"applied": True, "reason": "kv_compacted:per_head", "cache_len_after": 10}

    def batch(requests, scheduler_output):
        calls.append(("batch", [r for r, _ in requests]))
        return {r: {"applied": False, "reason": "under_budget", "cache_len_after": 5} for r, _ in requests}

    runner = types.SimpleNamespace(triattention_apply_compression=hook)
    ex = runner_actions.RunnerHookCompressionExecutor(runner)
    assert ex.execute("a", None, None).applied is True
    out = ex.execute_batch([("a", None), ("b", None)], None)          # no batch hook: falls back to the per-request hook
    assert [c[0] for c in calls] == ["one", "one", "one"] and out["b"].cache_len_after == 10
    runner.triattention_apply_compression_batch = batch
    out = ex.execute_batch([("a", None), ("b", None)], None)
    assert calls[-1] == ("batch", ["a", "b"]) and out["a"].reason == "under_budget" and out["a"].applied is False
    assert runner_actions.RunnerHookCompressionExecutor(types.SimpleNamespace()).execute("a", None, None).reason == "runner_hook_missing"


def test_state_store_follows_the_reference_call_by_call():
    """RequestStateStore against the reference's own snapshots (tests/golden/state_store_cases.json)."""
    import state_store_scenario as sss
    from triattention_b200.state import RequestStateStore

    want = json.loads((Path(__file__).resolve().parent / "golden" / "state_store_cases.json").read_text())
    got = json.loads(json.dumps(sss.replay(RequestStateStore())))
    assert len(got) == len(want) == len(sss.CALLS)
    for n, (g, w) in enumerate(zip(got, want)):
        assert g == w, (n, sss.CALLS[n])


def test_driver_with_the_real_state_store():
    """The driver's bookkeeping lands in the store: counts, steps, lengths and the de-duplication of the next step."""
    from triattention_b200.state import RequestStateStore
    import logging
    import types
    store = RequestStateStore()
    store.ensure("a", 100, False)
    store.mark_trigger("a", "length_threshold", 4)
    sig = CompressionSignal(req_id="a", should_compress=True, reason="length_threshold", estimated_cache_len=2177, step=4,
                            kv_usage=None, protect_prefill=False, prefill_len=100, scheduled_tokens=1)
    ex = ras.ScriptedExecutor({"a": ras.APPLIED}, runner_actions.CompressionExecutionResult)
    log = logging.getLogger("t")
    log.disabled = True
    so = types.SimpleNamespace(scheduled_cached_reqs=types.SimpleNamespace(req_ids=["a"], num_computed_tokens=[2176]))
    kw = dict(executor=ex, state_store=store, scheduler_output=so, strict_no_downgrade=False,
              allowed_strict_skip_reasons=set(), logger=log, log_decisions=False)
    ev = runner_actions.execute_runner_compression_actions(signals={"a": sig}, **kw)
    st = store.get("a")
    assert ev[0]["status"] == "applied" and st.compression_count == 1 and st.last_compression_step == 4
    assert st.current_cache_len == 2049 and st.last_absorbed_cache_len == 2048 and st.nct_at_last_compression == 2176
    # the scheduler repeats the signal one step later (batch-queue race): it must not run again
    again = CompressionSignal(req_id="a", should_compress=True, reason="length_threshold", estimated_cache_len=2178, step=5,
                              kv_usage=None, protect_prefill=False, prefill_len=100, scheduled_tokens=1)
    ev = runner_actions.execute_runner_compression_actions(signals={"a": again}, **kw)
    assert ev[0]["reason"] == "batch_queue_dedup" and ex.calls == ["a"] and store.get("a").compression_count == 1


def test_step_life_cycle_follows_the_reference():
    """Arrivals, departures, preemptions, signals and actions over four steps: events and store snapshots after each
    step equal the reference's (tests/golden/step_lifecycle_cases.json)."""
    import step_lifecycle_scenario as sls
    from triattention_b200.state import RequestStateStore

    want = json.loads((Path(__file__).resolve().parent / "golden" / "step_lifecycle_cases.json").read_text())
    got = json.loads(json.dumps(sls.replay(runner_actions, RequestStateStore(), CompressionSignal,
                                           runner_actions.CompressionExecutionResult)))
    assert len(got) == len(want)
    for n, (g, w) in enumerate(zip(got, want)):
        assert g == w, n


def test_legacy_estimate_switch_keeps_the_schedulers_length():
    """After a compression the worker counts the cache length itself; the legacy switch takes the scheduler's
    estimate instead (the reference's TRIATTN_RUNTIME_LEGACY_COMPRESSED_ESTIMATE)."""
    import logging
    import types
    from triattention_b200.state import RequestStateStore

    log = logging.getLogger("legacy_estimate")

    def run(legacy):
        store = RequestStateStore()
        store.ensure(req_id="a", prefill_len=10, protect_prefill=False)
        store.update_cache_len("a", 2177, step=1)
        store.mark_compressed("a", step=1, cache_len=2048)
        so = types.SimpleNamespace(triattention_step=2, triattention_signals={"a": CompressionSignal(
            req_id="a", should_compress=False, reason="none", estimated_cache_len=2178, step=2, kv_usage=None,
            protect_prefill=False, prefill_len=10, scheduled_tokens=1)})
        runner_actions.consume_runner_signals(state_store=store, scheduler_output=so, last_step=1, logger=log,
                                              log_decisions=False, legacy_compressed_estimate=legacy)
        return store.get("a").current_cache_len

    assert run(False) == 2049
    assert run(True) == 2178
    assert run(None) == (2178 if runner_actions.LEGACY_COMPRESSED_ESTIMATE else 2049)
