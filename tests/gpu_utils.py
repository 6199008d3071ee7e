"""Helpers shared by the GPU parity tests: move a CPU case to the device and drive the C ABI through ops."""
from __future__ import annotations

import torch

from triattention_b200 import _native, ops
import synth


def device_stats(stats: synth.SyntheticStats, offsets: torch.Tensor, freq_scale_sq=None, dev="cuda") -> ops.DeviceStats:
    fs = torch.ones_like(stats.q_abs_mean) if freq_scale_sq is None else freq_scale_sq
    return ops.DeviceStats(
        stats.q_mean_real.to(dev).contiguous(), stats.q_mean_imag.to(dev).contiguous(),
        stats.q_abs_mean.to(dev).contiguous(), fs.to(dev).contiguous(),
        stats.inv_freq.to(dev).contiguous(), offsets.to(dev).contiguous(),
        rope_interleaved=(stats.rope_style == "interleaved"))


def block_table_tensor(block_id_lists, dev="cuda") -> torch.Tensor:
    width = max(len(b) for b in block_id_lists)
    bt = torch.zeros((len(block_id_lists), width), dtype=torch.int32)
    for i, ids in enumerate(block_id_lists):
        bt[i, : len(ids)] = torch.as_tensor(ids, dtype=torch.int32)
    return bt.to(dev)


def raw_to_reference_layout(raw: torch.Tensor, g: int, T: int) -> torch.Tensor:
    """[L, B, Hkv, t_pad, Gp] -> [L, B, Hkv*g, T] (query head h = kvh*g + slot)."""
    L, B, Hkv, t_pad, gp = raw.shape
    return raw[:, :, :, :T, :g].permute(0, 1, 2, 4, 3).reshape(L, B, Hkv * g, T)


def score_tolerance_ok(got: torch.Tensor, ref: torch.Tensor, rtol: float = 1e-3):
    """max |got-ref| / max(|ref|, sigma_row) <= rtol, rows along the last axis. Returns (ok, worst)."""
    sigma = ref.std(dim=-1, keepdim=True)
    denom = torch.maximum(ref.abs(), sigma).clamp_min(1e-6)
    worst = float(((got - ref).abs() / denom).max())
    return worst <= rtol, worst


def keep_sets_match_modulo_near_ties(keep: torch.Tensor, ref_keep: torch.Tensor, ref_scores: torch.Tensor,
                                     rtol: float = 1e-3):
    """Rows equal as sets except for indices whose reference score is within rtol*sigma_row of the cut-off
    (the k-th largest reference score), the tie window of the score contract.

    Returns (ok, number_of_differing_indices).
    """
    diff_total = 0
    for r in range(keep.shape[0]):
        a = set(keep[r].tolist())
        b = set(ref_keep[r].tolist())
        if a == b:
            continue
        row = ref_scores[r]
        finite = row[torch.isfinite(row)]
        sigma = float(finite.std()) if finite.numel() > 1 else 1.0
        cutoff = float(row[ref_keep[r]].min())
        for idx in a ^ b:
            diff_total += 1
            if abs(float(row[idx]) - cutoff) > rtol * max(sigma, 1e-6):
                return False, diff_total
    return True, diff_total
