"""Rebuild the inputs of a golden case from its stored parameters (same generator as make_golden.py)."""
from __future__ import annotations

import torch

import synth


def build_paged_case(p: dict):
    """(stats, per-layer paged caches, block ids) regenerated from the parameter dict of a fixture."""
    gen = torch.Generator().manual_seed(int(p["seed"]))
    inv_freq = synth.rope_inv_freq(p["head_dim"], p["theta"], p.get("llama3"))
    stats = synth.make_stats(p["num_layers"], p["num_q_heads"], p["head_dim"], inv_freq, gen,
                             rope_style=p.get("rope_style", "half"))
    T = p["total_tokens"]
    bs = p["block_size"]
    nblk = (T + bs - 1) // bs
    nb_total = nblk + p.get("spare_blocks", 5)
    if p.get("consecutive_blocks", False):
        block_ids = list(range(2, 2 + nblk))
        nb_total = max(nb_total, 2 + nblk)
    else:
        block_ids = synth.random_block_ids(nblk, nb_total, gen)
    caches = []
    for _l in range(p["num_layers"]):
        cache = synth.make_paged_layer(nb_total, bs, p["num_kv_heads"], p["head_dim"], kv_axis=p["kv_axis"])
        k = synth.make_rotated_keys(p["num_kv_heads"], T, p["head_dim"], inv_freq, gen,
                                    rope_style=p.get("rope_style", "half"))
        v = synth.make_values(p["num_kv_heads"], T, p["head_dim"], gen)
        synth.write_tokens_to_paged(cache, p["kv_axis"], block_ids, bs, k, v)
        caches.append(cache)
    return stats, caches, block_ids


def build_real_stats_case(p: dict, arrays):
    """Inputs of the fixture that uses two layers of shipped Qwen3-8B statistics."""
    inv_freq = torch.from_numpy(arrays["inv_freq"])
    stats = synth.SyntheticStats(
        torch.from_numpy(arrays["q_mean_real"]), torch.from_numpy(arrays["q_mean_imag"]),
        torch.from_numpy(arrays["q_abs_mean"]), inv_freq, p["head_dim"], "half")
    gen = torch.Generator().manual_seed(int(p["seed"]))
    T, bs = p["total_tokens"], p["block_size"]
    nblk = (T + bs - 1) // bs
    block_ids = synth.random_block_ids(nblk, nblk + 7, gen)
    caches = []
    for _l in range(p["num_layers"]):
        cache = synth.make_paged_layer(nblk + 7, bs, p["num_kv_heads"], p["head_dim"], kv_axis=0)
        k = synth.make_rotated_keys(p["num_kv_heads"], T, p["head_dim"], inv_freq, gen)
        v = synth.make_values(p["num_kv_heads"], T, p["head_dim"], gen)
        synth.write_tokens_to_paged(cache, 0, block_ids, bs, k, v)
        caches.append(cache)
    return stats, caches, block_ids


def stats_by_layer(stats: synth.SyntheticStats, freq_scale_sq=None) -> dict:
    """{layer: dict of [Hs, F] tensors} as the checker's selection functions take them."""
    out = {}
    for l in range(stats.num_layers):
        fs = torch.ones_like(stats.q_abs_mean[l]) if freq_scale_sq is None else freq_scale_sq[l]
        out[l] = {
            "q_mean_real": stats.q_mean_real[l],
            "q_mean_imag": stats.q_mean_imag[l],
            "q_abs_mean": stats.q_abs_mean[l],
            "freq_scale_sq": fs,
        }
    return out


def build_stats_case(p: dict, inv_freq: torch.Tensor):
    """(per-layer paged caches, block ids) of a fixture whose statistics come from a file: K/V and the block order are
    drawn from the seed alone."""
    gen = torch.Generator().manual_seed(int(p["seed"]))
    T, bs = p["total_tokens"], p["block_size"]
    nblk = (T + bs - 1) // bs
    block_ids = synth.random_block_ids(nblk, nblk + 5, gen)
    caches = []
    for _l in range(p["num_layers"]):
        cache = synth.make_paged_layer(nblk + 5, bs, p["num_kv_heads"], p["head_dim"], kv_axis=0)
        synth.write_tokens_to_paged(cache, 0, block_ids, bs,
                                    synth.make_rotated_keys(p["num_kv_heads"], T, p["head_dim"], inv_freq, gen),
                                    synth.make_values(p["num_kv_heads"], T, p["head_dim"], gen))
        caches.append(cache)
    return caches, block_ids
