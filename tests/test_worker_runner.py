"""The worker's runner proxy against results of the reference's own runner on the same scripted inputs
(tests/golden/worker_runner_cases.json, written by tests/golden/make_golden.py --only worker_runner)."""
from __future__ import annotations

import json
import sys
import types
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

import worker_runner_scenarios as wrs  # noqa: E402
from triattention_b200 import worker_runner  # noqa: E402
from triattention_b200.config import TriAttentionRuntimeConfig  # noqa: E402
from triattention_b200.signals import CompressionSignal  # noqa: E402
from triattention_b200.state import RequestStateStore  # noqa: E402

WANT = json.loads((HERE / "golden" / "worker_runner_cases.json").read_text())


def _plain(x):
    return json.loads(json.dumps(x))


def _self_trigger(base_runner, config, store, so, signals, last_step):
    return worker_runner.supplement_worker_self_triggers(base_runner=base_runner, config=config, state_store=store,
                                                         scheduler_output=so, signals=signals, last_step=last_step)


@pytest.mark.parametrize("case", wrs.self_trigger_cases(CompressionSignal), ids=lambda c: c["name"])
def test_self_triggers_follow_the_reference(case):
    assert _plain(wrs.run_self_trigger(_self_trigger, RequestStateStore, case)) == WANT["self_trigger"][case["name"]]


@pytest.mark.parametrize("case", wrs.TRIM_CASES, ids=lambda c: c["name"])
def test_new_block_ids_are_trimmed_like_the_reference(case):
    def trim(base_runner, store, so):
        worker_runner.trim_new_block_ids_for_compressed_reqs(base_runner=base_runner, state_store=store,
                                                             scheduler_output=so)
    assert _plain(wrs.run_trim(trim, RequestStateStore, case)) == WANT["trim"][case["name"]]


@pytest.mark.parametrize("case", wrs.OVERRIDE_CASES, ids=lambda c: c["name"])
def test_overrides_of_a_step_follow_the_reference(case):
    got = wrs.run_overrides(worker_runner.prepare_effective_input_overrides,
                            worker_runner.needs_effective_input_overrides, RequestStateStore, case)
    assert _plain(got) == WANT["overrides"][case["name"]]


def test_events_are_attached_like_the_reference():
    assert _plain(wrs.run_attach(worker_runner)) == WANT["attach"]


def test_whole_steps_follow_the_reference():
    cfg = TriAttentionRuntimeConfig(kv_budget=64, divide_length=16, protect_prefill=False, log_decisions=False,
                                    enable_experimental_kv_compaction=True)
    got = _plain(wrs.run_steps(worker_runner.TriAttentionModelRunner, cfg, CompressionSignal))
    assert len(got) == len(WANT["steps"])
    for n, (g, w) in enumerate(zip(got, WANT["steps"])):
        assert g == w, n
    # not vacuous: an applied and a skipped event, events riding on the scheduler output, and a worker self-trigger
    assert [e["status"] for e in got[3]["events_on_output"]] == ["applied", "skipped"]
    assert got[7]["output"] is None and got[7]["events_on_scheduler_output"][0]["req_id"] == "a"
    assert got[8]["calls"][0] == ["hook", "c", 101, 1]


def test_overrides_are_published_while_the_engine_runs():
    """During the engine's execute_model the overrides of the step can be read; before and after there are none,
    and a step without compressed requests publishes nothing."""
    seen = []
    base = types.SimpleNamespace(
        requests={"a": types.SimpleNamespace(num_computed_tokens=201)},
        input_batch=types.SimpleNamespace(req_id_to_index={"a": 3}, block_table=None))

    def execute_model(scheduler_output, intermediate_tensors=None):
        seen.append(worker_runner.current_effective_input_overrides())
        return types.SimpleNamespace()

    base.execute_model = execute_model
    store = RequestStateStore()
    store.ensure(req_id="a", prefill_len=10, protect_prefill=False)
    so = types.SimpleNamespace(num_scheduled_tokens={"a": 1}, triattention_step=2,
                               scheduled_cached_reqs=types.SimpleNamespace(req_ids=["a"], num_computed_tokens=[201]))
    worker_runner.execute_base_model_with_effective_overrides(base_runner=base, state_store=store, scheduler_output=so)
    store.update_cache_len("a", 200, step=1)
    store.mark_compressed("a", step=1, cache_len=64, scheduled_tokens=1, scheduler_nct=200)
    so2 = types.SimpleNamespace(num_scheduled_tokens={"a": 1}, triattention_step=2,
                                scheduled_cached_reqs=types.SimpleNamespace(req_ids=["a"], num_computed_tokens=[201]))
    perf = {}
    worker_runner.execute_base_model_with_effective_overrides(base_runner=base, state_store=store, scheduler_output=so2,
                                                              perf_out=perf)
    assert seen[0] is None
    assert seen[1].seq_base_map == {3: 65} and seen[1].pos_delta_map == {3: -136}
    assert seen[1].expected_req_row_indices == (3,) and seen[1].expected_query_lens == (1,)
    assert worker_runner.current_effective_input_overrides() is None
    assert set(perf) == {"override_prep_ms", "base_exec_ms"}


def test_input_patch_is_installed_once_and_its_failure_is_fatal():
    calls = []
    base = types.SimpleNamespace(requests={}, input_batch=types.SimpleNamespace())
    cfg = TriAttentionRuntimeConfig(kv_budget=64, divide_length=16)
    proxy = worker_runner.TriAttentionModelRunner(base, cfg, install_runtime_input_patch=lambda: calls.append(1) or True)
    proxy._ensure_runtime_input_patch_if_needed(False)
    proxy._ensure_runtime_input_patch_if_needed(True)
    proxy._ensure_runtime_input_patch_if_needed(True)
    assert calls == [1]
    failing = worker_runner.TriAttentionModelRunner(base, cfg, install_runtime_input_patch=lambda: False)
    with pytest.raises(RuntimeError, match="patch installation failed"):
        failing._ensure_runtime_input_patch_if_needed(True)


def test_step_profile_line(monkeypatch):
    import logging
    from triattention_b200.perf_profile import TriAttentionPerfProfile

    monkeypatch.setenv("TRIATTN_RUNTIME_PERF_PROFILE", "1")
    monkeypatch.setenv("TRIATTN_RUNTIME_PERF_LOG_EVERY", "2")
    prof = TriAttentionPerfProfile.from_env(logging.getLogger("step_profile"))
    prof.record_compression_events([{"status": "applied"}, {"status": "skipped", "reason": "under_budget"},
                                    {"status": "error"}, "junk"])
    prof.record_model_output(types.SimpleNamespace(cudagraph_stats=types.SimpleNamespace(runtime_mode="FULL")))
    for trig in (True, False):
        prof.record_step(has_trigger=trig, uses_overrides=True, t_state_ms=1.0, t_compress_ms=2.0, t_reclaim_ms=3.0,
                         t_override_prep_ms=4.0, t_base_exec_ms=5.0, t_total_exec_ms=20.0)
    assert prof.summary_line() == (
        "TRIATTN_PERF steps=2 trig_steps=1 override_steps=2 compress_calls=3 applied=1 skipped=1 errors=1 "
        "avg_ms(total=20.00 state=1.00 compress=2.00 reclaim=3.00 override_prep=4.00 base_exec=5.00) "
        "top_skip_reasons=under_budget:1 cudagraph_modes={'FULL': 1}")


def test_worker_installs_the_proxy_with_the_first_signal(monkeypatch):
    """The engine's runner is left alone until a scheduler output carries TriAttention signals; then the hook is
    installed on it and it is wrapped (once), and the model directory is taken from the engine's model config."""
    monkeypatch.delenv("TRIATTN_DEBUG_EARLY_INSTALL_PROXY", raising=False)
    base = types.SimpleNamespace(requests={}, tag="engine runner")
    worker = types.SimpleNamespace(model_runner=base, model_config=types.SimpleNamespace(model=" /models/qwen3 "))
    cfg = TriAttentionRuntimeConfig(kv_budget=64, divide_length=16)
    worker_runner.prepare_worker(worker, cfg)
    assert worker.model_runner is base and worker._triattention_runner_proxy_installed is False
    assert str(cfg.model_path) == "/models/qwen3"
    calls = []
    run = lambda w, so: calls.append(type(w.model_runner).__name__) or "ran"
    assert worker_runner.worker_execute_model(worker, types.SimpleNamespace(triattention_signals={}), run) == "ran"
    assert worker.model_runner is base
    installed = []
    monkeypatch.setattr("triattention_b200.hook.install_runner_compression_hook",
                        lambda base_runner, config: installed.append((base_runner, config)))
    so = types.SimpleNamespace(triattention_signals={"a": object()})
    worker_runner.worker_execute_model(worker, so, run)
    worker_runner.worker_execute_model(worker, so, run)
    assert isinstance(worker.model_runner, worker_runner.TriAttentionModelRunner)
    assert worker.model_runner.tag == "engine runner"            # everything else passes through to the engine's runner
    assert installed == [(base, cfg)] and worker._triattention_runner_proxy_installed is True
    assert calls == ["SimpleNamespace", "TriAttentionModelRunner", "TriAttentionModelRunner"]
    # eager installation for debugging
    monkeypatch.setenv("TRIATTN_DEBUG_EARLY_INSTALL_PROXY", "1")
    other = types.SimpleNamespace(model_runner=types.SimpleNamespace(requests={}), model_config=None)
    worker_runner.prepare_worker(other, TriAttentionRuntimeConfig(kv_budget=64, divide_length=16, model_path="/m"))
    assert isinstance(other.model_runner, worker_runner.TriAttentionModelRunner)
