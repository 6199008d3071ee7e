"""Effective-length overrides after compaction: the numpy checker against outputs of the reference's own
helpers (CPU), and the CUDA kernel behind the reference's call signatures against the same fixtures (GPU)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import input_patch as chk

GOLDEN = Path(__file__).resolve().parent / "golden"
MANIFEST = json.loads((GOLDEN / "manifest.json").read_text())["input_patch_cases"]
CASES = sorted(MANIFEST["cases"])


@pytest.fixture(scope="module")
def data():
    return np.load(GOLDEN / MANIFEST["file"])


def _maps(data, name):
    keys = data[f"{name}/base_keys"].tolist()
    return (dict(zip(keys, data[f"{name}/base_vals"].tolist())), dict(zip(keys, data[f"{name}/delta_vals"].tolist())))


@pytest.mark.parametrize("name", CASES)
def test_checker_matches_reference_outputs(data, name):
    meta = MANIFEST["cases"][name]
    idx, qsl = data[f"{name}/idx_mapping"], data[f"{name}/query_start_loc"]
    base_map, delta_map = _maps(data, name)
    got = chk.seq_lens_from_effective_lengths(idx, qsl, data[f"{name}/dense_base"], data[f"{name}/seq_lens"])
    assert np.array_equal(got, data[f"{name}/seq_lens_dense_out"])
    ok, got = chk.seq_lens_from_effective_base_map(idx, qsl, base_map, data[f"{name}/seq_lens"])
    assert ok == meta["sparse_applied"]
    assert np.array_equal(got, data[f"{name}/seq_lens_sparse_out"])
    shifted = chk.shift_positions_from_sparse_deltas(idx, qsl, data[f"{name}/positions"], delta_map)
    assert (shifted is not None) == meta["shifted"]
    if shifted is not None:
        assert np.array_equal(shifted, data[f"{name}/positions_out"])


def test_checker_declines_like_the_reference():
    idx, qsl, pos = np.array([2, 0]), np.array([0, 2, 1]), np.arange(4)
    assert chk.shift_positions_from_sparse_deltas(idx, qsl, pos, {2: -3}) is None          # decreasing starts
    assert chk.shift_positions_from_sparse_deltas(idx, np.array([0, 0, 0]), pos, {2: -3}) is None  # no query tokens
    assert chk.shift_positions_from_sparse_deltas(idx, np.array([3, 4, 9]), pos, {0: -3}) is None  # leaves the buffer
    assert chk.seq_lens_from_effective_base_map(idx, np.array([0, 1, 2]), {}, np.zeros(2, np.int32))[0] is False


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_kernel_matches_reference_outputs(data, name):
    from triattention_b200 import input_patch_ops as ops
    meta = MANIFEST["cases"][name]
    dev = "cuda"
    idx = torch.from_numpy(data[f"{name}/idx_mapping"]).to(dev)
    qsl = torch.from_numpy(data[f"{name}/query_start_loc"]).to(dev)
    base_map, delta_map = _maps(data, name)
    seq = torch.from_numpy(data[f"{name}/seq_lens"]).to(dev)
    ops.overwrite_seq_lens_from_effective_lengths(idx_mapping=idx, query_start_loc=qsl,
                                                  effective_num_computed_tokens=torch.from_numpy(data[f"{name}/dense_base"]).to(dev),
                                                  seq_lens=seq)
    assert np.array_equal(seq.cpu().numpy(), data[f"{name}/seq_lens_dense_out"])
    seq = torch.from_numpy(data[f"{name}/seq_lens"]).to(dev)
    ok = ops.overwrite_seq_lens_from_effective_base_map(idx_mapping=idx, query_start_loc=qsl,
                                                        effective_base_by_req_idx=base_map, seq_lens=seq)
    assert ok == meta["sparse_applied"]
    assert np.array_equal(seq.cpu().numpy(), data[f"{name}/seq_lens_sparse_out"])
    positions = torch.from_numpy(data[f"{name}/positions"]).to(dev)
    shifted = ops.shift_positions_from_sparse_deltas(idx_mapping=idx, query_start_loc=qsl, positions=positions,
                                                     pos_delta_by_req_idx=delta_map)
    assert (shifted is not None) == meta["shifted"]
    if shifted is not None:
        assert np.array_equal(shifted.cpu().numpy(), data[f"{name}/positions_out"])
        assert np.array_equal(positions.cpu().numpy(), data[f"{name}/positions"])  # the input is not modified


@pytest.mark.gpu
def test_kernel_on_a_large_random_batch_against_checker():
    from triattention_b200 import input_patch_ops as ops
    rng = np.random.default_rng(7)
    R, rows = 3000, 5000
    idx = rng.permutation(rows)[:R].astype(np.int32)
    qlen = rng.integers(0, 6, R)
    qsl = np.concatenate([[0], np.cumsum(qlen)]).astype(np.int32)
    pos = rng.integers(0, 1 << 40, int(qsl[-1]) + 11)
    chosen = rng.choice(idx, 700, replace=False)
    base_map = {int(r): int(rng.integers(1, 1 << 20)) for r in chosen}
    delta_map = {int(r): -int(rng.integers(0, 5000)) for r in chosen}
    seq0 = rng.integers(1, 1 << 20, R + 5).astype(np.int32)
    ok_ref, seq_ref = chk.seq_lens_from_effective_base_map(idx, qsl, base_map, seq0)
    pos_ref = chk.shift_positions_from_sparse_deltas(idx, qsl, pos, delta_map)
    dev = "cuda"
    seq = torch.from_numpy(seq0).to(dev)
    ok = ops.overwrite_seq_lens_from_effective_base_map(idx_mapping=torch.from_numpy(idx).to(dev),
                                                        query_start_loc=torch.from_numpy(qsl).to(dev),
                                                        effective_base_by_req_idx=base_map, seq_lens=seq)
    assert ok == ok_ref and np.array_equal(seq.cpu().numpy(), seq_ref)
    out = ops.shift_positions_from_sparse_deltas(idx_mapping=torch.from_numpy(idx).to(dev),
                                                 query_start_loc=torch.from_numpy(qsl).to(dev),
                                                 positions=torch.from_numpy(pos).to(dev), pos_delta_by_req_idx=delta_map)
    assert out is not None and pos_ref is not None and np.array_equal(out.cpu().numpy(), pos_ref)
