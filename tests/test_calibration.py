"""Calibration arithmetic (un-rotate captured queries, per-head complex mean and mean magnitude) against outputs of
the reference's own helpers, and the statistics file it writes through the loader the scorer uses."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from triattention_b200 import calibration
from triattention_b200.stats import load_frequency_stats

GOLDEN = Path(__file__).resolve().parent / "golden"
MANIFEST = json.loads((GOLDEN / "manifest.json").read_text())["calibration_cases"]


@pytest.mark.parametrize("name", sorted(MANIFEST["cases"]))
def test_query_statistics_match_reference_helpers(name):
    meta = MANIFEST["cases"][name]
    data = np.load(GOLDEN / MANIFEST["file"])
    got = calibration.query_frequency_stats(torch.from_numpy(data[f"{name}/q_rot"]), torch.from_numpy(data[f"{name}/cos"]),
                                            torch.from_numpy(data[f"{name}/sin"]), meta["attn_scale"], meta["rope_style"])
    for key in ("q_mean_real", "q_mean_imag", "q_abs_mean"):
        ref = torch.from_numpy(data[f"{name}/{key}"])
        assert torch.allclose(got[key], ref, rtol=1e-5, atol=1e-6), key  # fp32 arithmetic in a different association


def test_written_file_loads_through_the_scorer_side_loader(tmp_path):
    gen = torch.Generator().manual_seed(5)
    H, T, D, L = 4, 19, 64, 3
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    cos, sin = calibration.rotary_tables(inv, T)
    layers = [calibration.query_frequency_stats(torch.randn((H, T, D), generator=gen), cos, sin) for _ in range(L)]
    path = tmp_path / "stats.pt"
    calibration.save_stats(path, layers, D, "half", inv_freq=inv, extra_metadata={"num_attention_heads": H, "num_layers": L})
    metadata, head_stats = load_frequency_stats(path, device="cpu", dtype=torch.float32)
    assert int(metadata["head_dim"]) == D and len(head_stats) == L
    for l in range(L):
        assert torch.equal(head_stats[l]["q_mean_complex"][..., 0], layers[l]["q_mean_real"])
        assert torch.equal(head_stats[l]["q_mean_complex"][..., 1], layers[l]["q_mean_imag"])
        assert torch.equal(head_stats[l]["q_abs_mean"], layers[l]["q_abs_mean"])
