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


def test_capture_query_stats_from_a_tiny_model():
    """Hooks on a small random Llama-style decoder: the captured, un-rotated statistics equal the plain per-head
    mean of q_proj(layer input) (rotating and un-rotating cancel), for plain and for Llama-3.1-scaled RoPE."""
    tf = pytest.importorskip("transformers")
    from triattention_b200 import calibration
    torch.manual_seed(0)
    try:
        cfg = tf.LlamaConfig(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256,
                             rope_parameters={"rope_type": "llama3", "rope_theta": 5e5, "factor": 8.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
        model = tf.LlamaForCausalLM(cfg).eval()
    except Exception as exc:  # another transformers generation
        pytest.skip(f"cannot build the tiny model here: {type(exc).__name__}")
    ids = torch.randint(0, 97, (1, 40))
    inputs = {}
    handles = [a.register_forward_pre_hook(lambda m, a_, k_, i=i: inputs.__setitem__(i, (a_[0] if a_ else k_["hidden_states"]).detach()),
                                           with_kwargs=True) for i, a in enumerate(calibration.find_attention_layers(model))]
    per_layer, info = calibration.capture_query_stats(model, ids)
    for h in handles:
        h.remove()
    assert info["head_dim"] == 16 and info["num_heads"] == 4 and len(per_layer) == 2
    for i, attn in enumerate(calibration.find_attention_layers(model)):
        q = attn.q_proj(inputs[i]).view(1, 40, 4, 16).transpose(1, 2)[0].detach()     # [H, T, D], un-rotated
        z = calibration.as_complex_pairs(q)
        assert torch.allclose(per_layer[i]["q_mean_real"], z.mean(1).real, atol=2e-5)
        assert torch.allclose(per_layer[i]["q_mean_imag"], z.mean(1).imag, atol=2e-5)
        assert torch.allclose(per_layer[i]["q_abs_mean"], z.abs().mean(1), atol=2e-5)
    assert info["inv_freq"] is not None and info["inv_freq"].numel() == 8
