"""The patched input-preparation wrappers against results of the reference's closures on the same scripted calls
(tests/golden/input_patch_closure_cases.json, written by tests/golden/make_golden.py --only input_patch_closures).
Cases that reach the CUDA kernel (sparse maps over several requests) run on the GPU; the others also on CPU."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

import input_patch_closure_scenarios as ipc  # noqa: E402
from triattention_b200 import input_patch, worker_runner  # noqa: E402

WANT = json.loads((HERE / "golden" / "input_patch_closure_cases.json").read_text())
NEEDS_KERNEL = {"sparse_bases_two_of_three", "sparse_base_for_a_row_not_in_the_batch", "slot_shift_sparse",
                "slot_shift_sparse_fails", "validation_passes"}


class _Api:
    make_prepare = staticmethod(input_patch.make_patched_prepare_pos_seq_lens)
    make_slots = staticmethod(input_patch.make_patched_compute_slot_mappings)
    consumed = staticmethod(worker_runner.effective_overrides_consumed)

    @staticmethod
    def scope(ov):
        return worker_runner.active_effective_input_overrides(worker_runner.EffectiveInputOverrides(**ov))


def _check(case, device):
    got = json.loads(json.dumps(ipc.run_case(_Api, case, device)))
    assert got == WANT[case["name"]]


@pytest.mark.parametrize("case", [c for c in ipc.CASES if c["name"] not in NEEDS_KERNEL], ids=lambda c: c["name"])
def test_wrappers_without_the_kernel(case):
    _check(case, "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("case", ipc.CASES, ids=lambda c: c["name"])
def test_wrappers_on_the_device(case):
    _check(case, "cuda")


def test_scope_flags_reset():
    ov = worker_runner.EffectiveInputOverrides(None, None, 5, 0)
    with worker_runner.active_effective_input_overrides(ov):
        assert not worker_runner.effective_overrides_consumed()
        worker_runner.mark_effective_overrides_consumed()
        worker_runner.assert_effective_overrides_consumed()
    assert not worker_runner.effective_overrides_consumed()
    with pytest.raises(RuntimeError, match="TRIATTN_EFFECTIVE_OVERRIDES_NOT_CONSUMED"):
        worker_runner.assert_effective_overrides_consumed()
