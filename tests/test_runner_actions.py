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
