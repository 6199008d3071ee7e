"""The two functions an engine patches over its input preparation so that a compressed request is attended over its
EFFECTIVE length: wrappers around the engine's ``prepare_pos_seq_lens`` and ``compute_slot_mappings`` with the
behaviour of the reference's ``runtime/input_patch_vllm_backend.py:105-244``, reading the overrides of the step from
``worker_runner.current_effective_input_overrides()`` and applying them with the CUDA kernel behind
``input_patch_ops``.

Outside an ``execute_model`` call with overrides both wrappers are a plain call of the original.  Inside one:
the sequence lengths the original computed are overwritten (one request: base + query length; several: the sparse
map, which must cover exactly the batch entries it names); positions stay in the absolute rotary space unless the
debug switch ``TRIATTN_DEBUG_ENABLE_SLOT_SHIFT=1`` asks for the shifted ones.  ``TRIATTN_RUNTIME_VALIDATE_MAPPING=1``
checks, once per step, that the batch rows and query lengths are the ones the overrides were built for.
"""
from __future__ import annotations

import os
from typing import Any, Callable

import torch

from . import input_patch_ops as _ops
from . import worker_runner as _wr

_TRUE = {"1", "true", "yes", "on"}


def _switch(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in _TRUE


def _validate_once(idx_mapping: torch.Tensor, query_start_loc: torch.Tensor, ov: Any) -> None:
    if os.environ.get("TRIATTN_RUNTIME_VALIDATE_MAPPING", "0") != "1" or _wr.mapping_validated():
        return
    num_reqs = int(idx_mapping.shape[0])
    if ov.expected_req_row_indices is not None:
        actual = idx_mapping.detach().to("cpu", dtype=torch.long).tolist()
        expected = [int(x) for x in ov.expected_req_row_indices]
        if actual != expected:
            raise RuntimeError(f"TRIATTN_IDX_MAPPING_MISMATCH:actual={actual}:expected={expected}")
    if ov.expected_query_lens is not None:
        expected = [int(x) for x in ov.expected_query_lens]
        if len(expected) != num_reqs:
            raise RuntimeError(f"TRIATTN_QUERY_LENS_COUNT_MISMATCH:expected_num_reqs={len(expected)}:"
                               f"actual_num_reqs={num_reqs}")
        qsl = query_start_loc[: num_reqs + 1].detach().to("cpu", dtype=torch.long)
        if qsl.numel() != num_reqs + 1:
            raise RuntimeError(f"TRIATTN_QUERY_START_LOC_SHAPE_INVALID:expected_numel={num_reqs + 1}:"
                               f"actual_numel={int(qsl.numel())}")
        lens = (qsl[1:] - qsl[:-1]).tolist()
        if any(n < 0 for n in lens):
            raise RuntimeError("TRIATTN_QUERY_START_LOC_NON_MONOTONIC")
        if lens != expected:
            raise RuntimeError(f"TRIATTN_QUERY_LENS_MISMATCH:actual={lens}:expected={expected}")
    _wr.mapping_validated(mark=True)


def make_patched_prepare_pos_seq_lens(original: Callable[..., None]) -> Callable[..., None]:
    def patched(idx_mapping, query_start_loc, num_computed_tokens, pos, seq_lens) -> None:
        ov = _wr.current_effective_input_overrides()
        if ov is None:
            original(idx_mapping, query_start_loc, num_computed_tokens, pos, seq_lens)
            return
        _wr.mark_effective_overrides_consumed()
        _validate_once(idx_mapping, query_start_loc, ov)
        original(idx_mapping, query_start_loc, num_computed_tokens, pos, seq_lens)
        if _switch("TRIATTN_DEBUG_DISABLE_SEQ_OVERRIDE"):
            return
        num_reqs = int(idx_mapping.shape[0])
        if num_reqs == 1 and ov.single_seq_base is not None:
            qlen = (query_start_loc[1] - query_start_loc[0]).to(device=seq_lens.device, dtype=seq_lens.dtype)
            seq_lens[0].copy_(qlen + int(ov.single_seq_base))  # stays on the device: no host read in the decode path
            return
        if ov.seq_base_map:
            done = _ops.overwrite_seq_lens_from_effective_base_map(
                idx_mapping=idx_mapping, query_start_loc=query_start_loc, effective_base_by_req_idx=ov.seq_base_map,
                seq_lens=seq_lens)
            if not done and num_reqs > 0:
                raise RuntimeError("TRIATTN_SEQ_LENS_SPARSE_BASE_APPLY_FAILED:"
                                   "sparse_base_present_but_no_rows_were_overwritten")

    return patched


def make_patched_compute_slot_mappings(original: Callable[..., Any]) -> Callable[..., Any]:
    def patched(self, idx_mapping, query_start_loc, positions):
        ov = _wr.current_effective_input_overrides()
        if ov is None:
            return original(self, idx_mapping, query_start_loc, positions)
        _wr.mark_effective_overrides_consumed()
        _validate_once(idx_mapping, query_start_loc, ov)
        if _switch("TRIATTN_DEBUG_DISABLE_SLOT_SHIFT") or not _switch("TRIATTN_DEBUG_ENABLE_SLOT_SHIFT"):
            return original(self, idx_mapping, query_start_loc, positions)
        num_reqs = int(idx_mapping.shape[0])
        if num_reqs == 1 and ov.single_pos_delta != 0:
            return original(self, idx_mapping, query_start_loc, positions.clone().add_(int(ov.single_pos_delta)))
        if ov.pos_delta_map:
            shifted = _ops.shift_positions_from_sparse_deltas(
                idx_mapping=idx_mapping, query_start_loc=query_start_loc, positions=positions,
                pos_delta_by_req_idx=ov.pos_delta_map)
            if shifted is not None:
                return original(self, idx_mapping, query_start_loc, shifted)
            if num_reqs > 0:
                raise RuntimeError("TRIATTN_SLOT_MAPPING_SPARSE_SHIFT_FAILED:"
                                   "sparse_pos_delta_present_but_shift_positions_failed")
        return original(self, idx_mapping, query_start_loc, positions)

    return patched
