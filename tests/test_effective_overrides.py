"""Effective-length overrides for the forward pass after a compaction: the builder against the reference's own
results (tests/golden/effective_override_cases.json, produced by runtime/effective_overrides.py:209-359), and its
output through the device kernel that applies it."""
from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

import effective_override_scenarios as eos
from triattention_b200 import effective_overrides as eo

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "effective_override_cases.json").read_text())


@pytest.mark.parametrize("sc", eos.scenarios(), ids=lambda sc: sc["name"])
def test_builder_reproduces_the_reference(sc):
    assert json.loads(json.dumps(eos.run_scenario(eo.build_effective_sparse_overrides, sc))) == GOLDEN[sc["name"]]


def test_result_is_remembered_on_the_scheduler_output():
    sc = next(s for s in eos.scenarios() if s["name"] == "stable_anchor_two_requests")
    runner, store, so = eos.build_inputs(sc)
    first = eo.build_effective_sparse_overrides(base_runner=runner, state_store=store, scheduler_output=so)
    store._states.clear()   # a second call in the same step must not recompute
    again = eo.build_effective_sparse_overrides(base_runner=runner, state_store=store, scheduler_output=so)
    assert again is first
    other_store = eos._Store({}, False)
    other = eo.build_effective_sparse_overrides(base_runner=runner, state_store=other_store, scheduler_output=so)
    assert other == eo.NO_OVERRIDES and other is not first   # another store has its own entry
    assert eo.scheduled_token_items(so) is eo.scheduled_token_items(so)
    assert eo.scheduled_token_items(None) == []


def test_row_lookup_order():
    import types
    r = types.SimpleNamespace(req_states=types.SimpleNamespace(req_id_to_index={}),
                              input_batch=types.SimpleNamespace(req_id_to_index={"a": 4}))
    assert eo.req_id_to_index(r) == {"a": 4}
    r = types.SimpleNamespace(input_batch=types.SimpleNamespace(_req_ids=["x", None, "y"]))
    assert eo.req_id_to_index(r) == {"x": 0, "y": 2}
    assert eo.req_id_to_index(types.SimpleNamespace()) is None


@pytest.mark.gpu
def test_overrides_flow_into_the_device_kernel():
    """Store -> builder -> input_patch_ops on the GPU: seq_lens of a compressed request follow its effective length."""
    import types
    from triattention_b200 import input_patch_ops
    from triattention_b200.state import RequestStateStore

    store = RequestStateStore()
    store.ensure("a", 100, False)
    store.ensure("b", 50, False)
    store.mark_compressed("a", step=3, cache_len=2048, scheduled_tokens=1, scheduler_nct=2175)
    runner = types.SimpleNamespace(requests={"a": types.SimpleNamespace(num_computed_tokens=2180),
                                             "b": types.SimpleNamespace(num_computed_tokens=700)},
                                   req_states=types.SimpleNamespace(req_id_to_index={"a": 1, "b": 0}))
    so = types.SimpleNamespace(num_scheduled_tokens={"a": 1, "b": 1},
                               scheduled_cached_reqs=types.SimpleNamespace(req_ids=["a", "b"], num_computed_tokens=[2180, 700]))
    seq_bases, pos_deltas, one_seq, one_delta = eo.build_effective_sparse_overrides(
        base_runner=runner, state_store=store, scheduler_output=so)
    assert seq_bases == {1: 2053} and pos_deltas == {1: -127} and one_seq == 2053 and one_delta == -127
    idx_mapping = torch.tensor([0, 1], dtype=torch.int32, device="cuda")        # batch row -> request-state row
    query_start_loc = torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda")
    seq_lens = torch.tensor([701, 2181], dtype=torch.int32, device="cuda")
    ok = input_patch_ops.overwrite_seq_lens_from_effective_base_map(
        seq_lens=seq_lens, idx_mapping=idx_mapping, query_start_loc=query_start_loc, effective_base_by_req_idx=seq_bases)
    assert ok and seq_lens.tolist() == [701, 2054]
