"""The pieces either side of the compression step, chained as an engine would chain them, on CPU with a scripted
hook: scheduler (tracker -> planner -> signals) -> worker (consume signals -> execute actions -> events) ->
scheduler (block-pool reclaim, allocation offset).  One request decodes 120 tokens past its prompt with a budget of
64 tokens and a slack of 16; every number below follows from those three."""
from __future__ import annotations

import logging
import types

from triattention_b200 import runner_actions, scheduler_side
from triattention_b200.layout_engine import truncate_tail_reclaim_group
from triattention_b200.plan_models import PlacementPlan, ReclaimEvent
from triattention_b200.state import RequestStateStore

BS, BUDGET, SLACK, PROMPT = 16, 64, 16, 70


class _Block:
    def __init__(self, block_id):
        self.block_id, self.block_hash = block_id, None


class _Pool:
    def __init__(self):
        self.freed, self.next_id = [], 0

    def take(self):
        self.next_id += 1
        return _Block(self.next_id - 1)

    def free_blocks(self, blocks):
        self.freed.append([b.block_id for b in blocks])


class _Hook:
    """What the installed hook reports for a request it compacts to the budget (hook result of a PlacementPlan)."""

    def __init__(self, worker_blocks):
        self.worker_blocks = worker_blocks

    def execute(self, req_id, signal, scheduler_output):
        ids = self.worker_blocks[req_id]
        kept, _removed, group = truncate_tail_reclaim_group(gid=0, normalized_block_ids=ids, cache_len_after=BUDGET,
                                                            block_size=BS)
        self.worker_blocks[req_id] = kept
        d = PlacementPlan(cache_len_after=BUDGET, selector_status="enabled", selection_mode="per_head",
                          effective_tokens_before=signal.estimated_cache_len, budget_total=BUDGET,
                          recent_unabsorbed_tokens=None,
                          block_reclaim=ReclaimEvent("truncate_tail", [group]) if group else None).to_hook_result_dict()
        return runner_actions.CompressionExecutionResult(applied=True, reason=d["reason"], cache_len_after=BUDGET,
                                                         details=d)


def test_trigger_compress_reclaim_loop():
    log = logging.getLogger("step_loop")
    log.disabled = True
    cfg = types.SimpleNamespace(kv_budget=BUDGET, divide_length=SLACK, protect_prefill=False,
                                include_prefill_in_budget=False, enable_kv_usage_trigger=False, kv_usage_trigger=0.98,
                                kv_usage_release=0.9, enable_experimental_block_reclaim=True,
                                require_physical_reclaim=True)
    pool = _Pool()
    manager = types.SimpleNamespace(req_to_blocks={"r": []}, num_cached_block={}, block_pool=pool)
    request = types.SimpleNamespace(num_computed_tokens=0)
    sched = types.SimpleNamespace(
        kv_cache_manager=types.SimpleNamespace(coordinator=types.SimpleNamespace(single_type_managers=[manager])),
        block_size=BS, requests={"r": request}, _effective_len_tracker=scheduler_side.EffectiveCacheLenTracker(),
        triattention_config=cfg)
    planner = scheduler_side.CompressionPlanner(cfg)
    store = RequestStateStore()
    worker_blocks = {"r": []}
    hook = _Hook(worker_blocks)
    triggers, last_step = [], 0
    for step in range(1, 122):
        n_new = PROMPT if step == 1 else 1
        # ---- scheduler: blocks for the tokens of this step, then the trigger decision
        effective = sched._effective_len_tracker.observe_num_computed("r", request.num_computed_tokens)
        while len(manager.req_to_blocks["r"]) * BS < effective + n_new:
            manager.req_to_blocks["r"].append(pool.take())
        signal = planner.build_signal("r", effective + n_new, PROMPT, step, scheduled_tokens=n_new)
        so = types.SimpleNamespace(triattention_step=step, triattention_signals={"r": signal},
                                   scheduled_new_reqs=[], finished_req_ids=[])
        # ---- worker: same block list as the scheduler's (plus what the scheduler appended), state store, actions
        worker_blocks["r"] = [b.block_id for b in manager.req_to_blocks["r"]]
        last_step, signals = runner_actions.consume_runner_signals(state_store=store, scheduler_output=so,
                                                                   last_step=last_step, logger=log, log_decisions=False)
        events = runner_actions.execute_runner_compression_actions(
            executor=hook, state_store=store, scheduler_output=so, signals=signals, strict_no_downgrade=True,
            allowed_strict_skip_reasons=set(), logger=log, log_decisions=False)
        request.num_computed_tokens += n_new
        # ---- scheduler: the worker's events come back with the step's output
        scheduler_side.apply_compression_events(sched, events)
        if events:
            assert [e["status"] for e in events] == ["applied"]
            triggers.append(step)
            assert [b.block_id for b in manager.req_to_blocks["r"]] == worker_blocks["r"]
            assert len(worker_blocks["r"]) == BUDGET // BS
            assert sched._effective_len_tracker.snapshot()["r"] == (BUDGET, request.num_computed_tokens)
            assert getattr(request, scheduler_side.EFFECTIVE_KV_OFFSET_ATTR) == request.num_computed_tokens - BUDGET
            # the compression ran before the step's token was written: the worker counts it on top of the budget
            assert store.get("r").current_cache_len == BUDGET + n_new
    # first trigger when prompt + decoded tokens reach budget + slack = 80 (step 11: 70 + 10), then every 16 tokens
    assert triggers == [11, 27, 43, 59, 75, 91, 107]
    assert store.get("r").compression_count == len(triggers)
    # each trigger gave back the fifth block (65..80 tokens need 5 blocks, 64 need 4), last block first
    assert all(len(f) == 1 for f in pool.freed) and len(pool.freed) == len(triggers)
    assert scheduler_side.prepare_request_effective_num_computed(request) == \
        sched._effective_len_tracker.observe_num_computed("r", request.num_computed_tokens)


def test_loop_through_the_top_level_entry_points():
    """The same request through ``schedule_with_signals`` -> ``TriAttentionModelRunner.execute_model`` ->
    ``update_from_output_with_events``: the entry points an engine binds, nothing called in between."""
    from triattention_b200 import worker_runner
    from triattention_b200.config import TriAttentionRuntimeConfig

    cfg = TriAttentionRuntimeConfig(kv_budget=BUDGET, divide_length=SLACK, window_size=8, log_decisions=False)
    pool = _Pool()
    pool.num_gpu_blocks = 1000
    manager = types.SimpleNamespace(req_to_blocks={"r": []}, num_cached_block={}, block_pool=pool)
    request = types.SimpleNamespace(num_computed_tokens=0, num_prompt_tokens=PROMPT)
    sched = types.SimpleNamespace(
        kv_cache_manager=types.SimpleNamespace(coordinator=types.SimpleNamespace(single_type_managers=[manager]),
                                               block_pool=pool, usage=0.1),
        block_size=BS, requests={"r": request}, running=[request], max_num_scheduled_tokens=8192)
    scheduler_side.attach_scheduler_state(sched, cfg)

    worker_blocks = {"r": []}
    hook = _Hook(worker_blocks)
    base_runner = types.SimpleNamespace(requests={"r": types.SimpleNamespace(num_computed_tokens=0)})
    base_runner.triattention_apply_compression = lambda req_id, signal, scheduler_output: \
        hook.execute(req_id, signal, scheduler_output).details
    base_runner.execute_model = lambda scheduler_output, intermediate_tensors=None: types.SimpleNamespace()
    proxy = worker_runner.TriAttentionModelRunner(base_runner, cfg)

    def base_schedule(s):
        n_new = PROMPT if s._triattention_step == 0 else 1
        held = getattr(request, scheduler_side.EFFECTIVE_NUM_COMPUTED_ATTR, None)
        held = request.num_computed_tokens if held is None else held      # what the allocation patch would use
        while len(manager.req_to_blocks["r"]) * BS < held + n_new:
            manager.req_to_blocks["r"].append(pool.take())
        new = [types.SimpleNamespace(req_id="r", num_computed_tokens=0, prompt_token_ids=[0] * PROMPT)] if n_new > 1 else []
        return types.SimpleNamespace(num_scheduled_tokens={"r": n_new}, scheduled_new_reqs=new, finished_req_ids=[],
                                     scheduled_cached_reqs=None)

    triggers = []
    for step in range(1, 122):
        so = scheduler_side.schedule_with_signals(sched, base_schedule)
        worker_blocks["r"] = [b.block_id for b in manager.req_to_blocks["r"]]
        base_runner.requests["r"].num_computed_tokens = request.num_computed_tokens
        output = proxy.execute_model(so)
        request.num_computed_tokens += so.num_scheduled_tokens["r"]
        scheduler_side.update_from_output_with_events(sched, so, output, lambda s, a, b: {})
        if output.triattention_compression_events:
            triggers.append(step)
            assert [b.block_id for b in manager.req_to_blocks["r"]] == worker_blocks["r"]
            assert len(worker_blocks["r"]) == BUDGET // BS
    # The first trigger is the scheduler's (70 + 10 tokens = budget + slack).  Later ones are the worker's own: its
    # count starts at budget + 1 after a compression (the step's token is already in) and the self-trigger adds the
    # step's token once more, so it fires two steps before the scheduler would - every 14 steps, as in the reference.
    assert triggers == [11, 25, 39, 53, 67, 81, 95, 109]
    assert proxy.snapshot_states()["r"].compression_count == len(triggers)
    assert len(pool.freed) == len(triggers)
    # the tracker last looked at the request when step 121 was scheduled: 120 steps done, the last compaction in step 109
    assert sched._effective_len_tracker.snapshot()["r"] == (BUDGET + 120 - triggers[-1], request.num_computed_tokens - 1)
