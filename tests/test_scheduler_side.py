"""Scheduler-side pieces (trigger planner, effective-length tracker, allocation-sync attributes, block-pool reclaim)
against results of the reference's own code on the same scripted inputs (tests/golden/scheduler_side_cases.json,
written by tests/golden/make_golden.py --only scheduler_side)."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

import scheduler_side_scenarios as sss  # noqa: E402
from triattention_b200 import scheduler_side  # noqa: E402

WANT = json.loads((HERE / "golden" / "scheduler_side_cases.json").read_text())


def _plain(x):
    return json.loads(json.dumps(x))


def test_trigger_planner_follows_the_reference():
    got = _plain(sss.replay_planner(scheduler_side.CompressionPlanner))
    assert sorted(got) == sorted(WANT["planner"])
    for name in got:
        for n, (g, w) in enumerate(zip(got[name], WANT["planner"][name])):
            assert g == w, (name, n)
    # the cases cover both triggers, the latch (armed at 0.95, still armed at 0.7, released at 0.5) and its priority
    reasons = {s["reason"] for sigs in got.values() for s in sigs}
    assert reasons == {"none", "length_threshold", "kv_usage_threshold"}
    pool = got["pool_pressure"]
    assert [s["should_compress"] for s in pool[2:7]] == [True, True, False, False, False]


def test_effective_length_tracker_follows_the_reference():
    got = _plain(sss.replay_tracker(scheduler_side.EffectiveCacheLenTracker()))
    assert len(got) == len(WANT["tracker"])
    for n, (g, w) in enumerate(zip(got, WANT["tracker"])):
        assert g == w, n


def test_allocation_sync_attributes_follow_the_reference():
    got = _plain(sss.replay_allocation_sync(scheduler_side))
    assert len(got) == len(WANT["allocation_sync"])
    for n, (g, w) in enumerate(zip(got, WANT["allocation_sync"])):
        assert g == w, n


@pytest.mark.parametrize("case", sss.RECLAIM_CASES, ids=[c["name"] for c in sss.RECLAIM_CASES])
def test_block_pool_reclaim_follows_the_reference(case):
    got = _plain(sss.run_reclaim_case(scheduler_side.apply_compression_events, scheduler_side.EffectiveCacheLenTracker,
                                      case))
    want = WANT["reclaim"][case["name"]]
    assert got == want
    if case["name"].startswith("error_"):
        assert got["error"] and got["error"].startswith("TriAttention block reclaim")


def test_reclaim_cases_exercise_the_pool():
    """The fixtures are not vacuous: blocks are freed last-first, hashed ones are evicted first, appended blocks stay."""
    two = WANT["reclaim"]["explicit_payload_two_groups"]
    assert two["pool_calls"] == [["evict", 0, 230], ["evict", 0, 236], ["free", 0, list(range(236, 227, -1))],
                                 ["free", 1, list(range(636, 627, -1))]]
    assert two["offsets"] == {"a": 2177 - 2048}
    late = WANT["reclaim"]["blocks_appended_after_the_hook"]
    assert late["blocks"][0]["a"] == list(range(128)) + [137, 138, 139]
    assert late["pool_calls"] == [["free", 0, list(range(136, 127, -1))]]
    assert WANT["reclaim"]["no_payload_during_prefill"]["pool_calls"] == []
    assert WANT["reclaim"]["payload_misses_a_group"]["blocks"][1]["a"] == list(range(300, 428))


class _StepApi:
    attach = staticmethod(scheduler_side.attach_scheduler_state)
    schedule = staticmethod(scheduler_side.schedule_with_signals)
    update = staticmethod(scheduler_side.update_from_output_with_events)


@pytest.mark.parametrize("name", sorted(sss.STEP_CONFIGS))
def test_scheduler_steps_follow_the_reference(name):
    """Eight scheduling steps (chunked prefill, decode, a trigger, events returning on the runner's output and on the
    scheduler output, a resumed and two finished requests) through schedule / update_from_output."""
    got = _plain(sss.run_scheduler_steps(_StepApi, sss.STEP_CONFIGS[name]))
    want = WANT["steps"][name]
    assert len(got) == len(want)
    for n, (g, w) in enumerate(zip(got, want)):
        assert g == w, (name, n)


def test_scheduler_step_fixtures_are_not_vacuous():
    steps = WANT["steps"]["length_trigger"]
    assert steps[3]["signals"]["a"]["should_compress"] and steps[3]["signals"]["a"]["estimated_cache_len"] == 80
    assert steps[3]["pool_calls"] == [["free", 0, [5, 4]]] and steps[3]["usage_in_stats"] == 0.7
    assert steps[4]["signals"]["a"]["estimated_cache_len"] == 66 and not steps[4]["signals"]["a"]["should_compress"]
    assert steps[4]["effective_markers"]["a"] == 65
    assert WANT["steps"]["small_pool_caps_the_step"][0]["cap_seen"] == 16
    assert all(s["cap_after"] == 8192 for s in WANT["steps"]["small_pool_caps_the_step"])
    assert WANT["steps"]["pool_pressure_trigger"][1]["signals"]["b"]["reason"] == "kv_usage_threshold"
    assert WANT["steps"]["compression_disabled"][3]["signals"] == {}


@pytest.mark.parametrize("case", sss.ALLOC_CASES, ids=lambda c: c["name"])
def test_slot_allocation_sees_the_effective_length(case):
    got = _plain(sss.run_alloc_case(scheduler_side.allocate_slots_with_effective_length, case))
    assert got == WANT["alloc"][case["name"]]


def test_boundary_predicates_follow_the_reference():
    from triattention_b200.signals import CompressionSignal

    got = sss.run_boundary_predicates(scheduler_side.scheduler_output_has_compression_boundary,
                                      scheduler_side.batch_queue_has_pending_compression_boundary, CompressionSignal)
    assert got == WANT["boundary"]
    assert WANT["alloc"]["offset_applied"]["seen"] == {"args": ["extra"], "computed": 380, "num_new": 7,
                                                       "kwargs": {"delay_cache_blocks": True, "x": 1}}
