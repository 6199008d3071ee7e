"""Scripted calls of the two patched input-preparation functions (sequence lengths, slot-mapping positions) with and
without active overrides, debug switches and the optional mapping validation.  The fixture generator runs them on the
reference's closures with CPU tensors, the GPU test on this package's with device tensors."""
from __future__ import annotations

import os

import torch

ENV_NAMES = ("TRIATTN_DEBUG_DISABLE_SEQ_OVERRIDE", "TRIATTN_DEBUG_DISABLE_SLOT_SHIFT", "TRIATTN_DEBUG_ENABLE_SLOT_SHIFT",
             "TRIATTN_RUNTIME_VALIDATE_MAPPING")

_NONE = dict(seq_base_map=None, pos_delta_map=None, single_seq_base=None, single_pos_delta=0,
             expected_req_row_indices=None, expected_query_lens=None)


def _ov(**kw):
    return {**_NONE, **kw}


# batch: idx_mapping (request-state rows), query lengths, num_computed_tokens per request-state row
BATCH3 = dict(idx=[4, 1, 6], qlens=[1, 3, 1], computed=[0, 300, 0, 0, 200, 0, 500, 0])
BATCH1 = dict(idx=[2], qlens=[1], computed=[0, 0, 950])

CASES = [
    dict(name="no_overrides_active", batch=BATCH3, overrides=None),
    dict(name="one_request_single_base", batch=BATCH1, overrides=_ov(seq_base_map={2: 64}, pos_delta_map={2: -886},
                                                                     single_seq_base=64, single_pos_delta=-886)),
    dict(name="sparse_bases_two_of_three", batch=BATCH3,
         overrides=_ov(seq_base_map={4: 64, 6: 70}, pos_delta_map={4: -136, 6: -430})),
    dict(name="sparse_base_for_a_row_not_in_the_batch", batch=BATCH3, overrides=_ov(seq_base_map={4: 64, 7: 70})),
    dict(name="seq_override_switched_off", batch=BATCH3, env={"TRIATTN_DEBUG_DISABLE_SEQ_OVERRIDE": "1"},
         overrides=_ov(seq_base_map={4: 64})),
    dict(name="slot_shift_single", batch=BATCH1, env={"TRIATTN_DEBUG_ENABLE_SLOT_SHIFT": "1"},
         overrides=_ov(seq_base_map={2: 64}, pos_delta_map={2: -886}, single_seq_base=64, single_pos_delta=-886)),
    dict(name="slot_shift_sparse", batch=BATCH3, env={"TRIATTN_DEBUG_ENABLE_SLOT_SHIFT": "1"},
         overrides=_ov(seq_base_map={4: 64, 1: 100}, pos_delta_map={4: -136, 1: -200})),
    dict(name="slot_shift_sparse_fails", batch=BATCH3, env={"TRIATTN_DEBUG_ENABLE_SLOT_SHIFT": "1"},
         overrides=_ov(pos_delta_map={4: -136, 7: -5})),
    dict(name="slot_shift_enabled_and_disabled", batch=BATCH1,
         env={"TRIATTN_DEBUG_ENABLE_SLOT_SHIFT": "1", "TRIATTN_DEBUG_DISABLE_SLOT_SHIFT": "1"},
         overrides=_ov(pos_delta_map={2: -886}, single_pos_delta=-886)),
    dict(name="validation_passes", batch=BATCH3, env={"TRIATTN_RUNTIME_VALIDATE_MAPPING": "1"},
         overrides=_ov(seq_base_map={4: 64}, expected_req_row_indices=(4, 1, 6), expected_query_lens=(1, 3, 1))),
    dict(name="validation_rows_differ", batch=BATCH3, env={"TRIATTN_RUNTIME_VALIDATE_MAPPING": "1"},
         overrides=_ov(seq_base_map={4: 64}, expected_req_row_indices=(4, 6, 1), expected_query_lens=(1, 3, 1))),
    dict(name="validation_query_lens_differ", batch=BATCH3, env={"TRIATTN_RUNTIME_VALIDATE_MAPPING": "1"},
         overrides=_ov(seq_base_map={4: 64}, expected_req_row_indices=(4, 1, 6), expected_query_lens=(1, 1, 1))),
    dict(name="validation_count_differs", batch=BATCH3, env={"TRIATTN_RUNTIME_VALIDATE_MAPPING": "1"},
         overrides=_ov(seq_base_map={4: 64}, expected_query_lens=(1, 3))),
]


def run_case(api, case, device) -> dict:
    """``api.make_prepare(original)``, ``api.make_slots(original)``, ``api.scope(overrides dict) -> context manager``,
    ``api.consumed() -> bool`` (valid inside the scope)."""
    b = case["batch"]
    idx = torch.tensor(b["idx"], dtype=torch.int32, device=device)
    qsl = torch.tensor([0] + list(torch.tensor(b["qlens"]).cumsum(0).tolist()), dtype=torch.int32, device=device)
    computed = torch.tensor(b["computed"], dtype=torch.int32, device=device)
    n_tok = int(qsl[-1])
    seen = {}

    def orig_prepare(idx_mapping, query_start_loc, num_computed_tokens, pos, seq_lens):
        n = int(idx_mapping.shape[0])
        ql = (query_start_loc[1:n + 1] - query_start_loc[:n]).to(seq_lens.dtype)
        seq_lens[:n] = num_computed_tokens[idx_mapping.long()].to(seq_lens.dtype) + ql

    def orig_slots(self, idx_mapping, query_start_loc, positions):
        seen["positions"] = positions.detach().to("cpu", dtype=torch.long).tolist()
        return "slots"

    prepare, slots = api.make_prepare(orig_prepare), api.make_slots(orig_slots)
    seq_lens = torch.zeros(len(b["idx"]) + 2, dtype=torch.int32, device=device)
    pos = torch.zeros(n_tok, dtype=torch.int64, device=device)
    positions = torch.cat([torch.arange(int(computed[r]), int(computed[r]) + q) for r, q in zip(b["idx"], b["qlens"])]
                          ).to(device=device, dtype=torch.int64)
    saved = {k: os.environ.get(k) for k in ENV_NAMES}
    for k in ENV_NAMES:
        os.environ.pop(k, None)
    os.environ.update(case.get("env", {}))
    out = {"prepare_error": None, "slots_error": None, "slots_returned": None, "consumed": None}
    try:
        def body():
            try:
                prepare(idx, qsl, computed, pos, seq_lens)
            except RuntimeError as exc:
                out["prepare_error"] = str(exc)
            try:
                out["slots_returned"] = slots(None, idx, qsl, positions)
            except RuntimeError as exc:
                out["slots_error"] = str(exc)
            out["consumed"] = api.consumed()

        if case["overrides"] is None:
            body()
        else:
            with api.scope(case["overrides"]):
                body()
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    out["seq_lens"] = seq_lens.detach().to("cpu").tolist()
    out["positions_given_to_the_engine"] = seen.get("positions")
    out["positions_untouched"] = positions.detach().to("cpu").tolist()
    return out
