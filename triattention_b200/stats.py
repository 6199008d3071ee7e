"""Loader of the per-layer Q/K frequency statistics (.pt) and packing for the kernels.

Accepts the two on-disk formats of the reference (core/utils.py:18-134):

* "R-KV" files written by the calibration script (scripts/calibrate.py:231-271):
  ``{"metadata": {head_dim, rope_style, sampled_heads, [inv_freq], ...},
  "stats": {"layerLL_headHH": {q_mean_real, q_mean_imag, q_abs_mean}}}``;
* "TriAttention" files with ``layer_stats[layer] = {q_mean_complex [H,F,2], freq_scale_sq [H,F], ...}``.

``inv_freq`` is taken from the metadata when present; otherwise it is derived
from ``rope_theta`` (default 10000, core/compressor.py:186-191).  The reference
may additionally fetch a model config from the Hub; that network path is not
reproduced - put ``inv_freq`` in the metadata for scaled-RoPE models.
"""
from __future__ import annotations

import re
from pathlib import Path
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import ops

_KEY = re.compile(r"^layer(\d+)_head(\d+)$")


def compute_rope_frequencies(head_dim: int, rope_theta: float = 10000.0, device="cpu") -> torch.Tensor:
    """``1 / theta^(2i/head_dim)`` as fp32 ``[head_dim/2]`` (core/utils.py:520-542)."""
    if head_dim % 2 != 0:
        raise ValueError(f"head_dim must be even, got {head_dim}")
    return 1.0 / (rope_theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))


def _inv_freq_from(metadata: dict, freq_count: int, device) -> Optional[torch.Tensor]:
    raw = metadata.get("inv_freq")
    if isinstance(raw, torch.Tensor):
        t = raw.to(device=device, dtype=torch.float32)
    elif isinstance(raw, (list, tuple)):
        t = torch.tensor(raw, device=device, dtype=torch.float32)
    else:
        return None
    if t.numel() < freq_count:
        raise ValueError(
            f"metadata.inv_freq has fewer elements than required by head_dim={2 * freq_count}: "
            f"got {t.numel()}, expected at least {freq_count}")
    return t[:freq_count].contiguous()


def _convert_rkv(stats: dict, device, dtype, num_kv_heads: Optional[int]) -> Tuple[dict, dict]:
    """Per-head flat records -> per-layer stacked tensors, with the optional GQA mean (core/utils.py:137-361)."""
    meta_in = stats.get("metadata", {}) or {}
    recs = stats.get("stats", {})
    layers, heads = set(), set()
    for key in recs:
        m = _KEY.match(key)
        if m:
            layers.add(int(m.group(1)))
            heads.add(int(m.group(2)))
    num_layers, num_heads = len(layers), len(heads)
    head_dim = int(meta_in.get("head_dim", 128))
    F = head_dim // 2
    if num_kv_heads is None:
        num_kv_heads = num_heads
    ratio = num_heads // num_kv_heads if num_kv_heads > 0 else 1
    metadata = {
        "num_attention_heads": num_heads,
        "num_kv_heads": num_kv_heads,
        "head_dim": head_dim,
        "num_layers": num_layers,
        "rope_style": meta_in.get("rope_style", "half"),
        "rope_type": meta_in.get("rope_type"),
        "rope_theta": meta_in.get("rope_theta", 10000.0),
        "gqa_ratio": ratio,
        "rkv_metadata": meta_in,
    }
    inv_freq = _inv_freq_from(meta_in, F, device)
    if inv_freq is not None:
        metadata["inv_freq"] = inv_freq
    head_stats: Dict[int, dict] = {}
    for layer in sorted(layers):
        q_abs, q_re, q_im = [], [], []
        for head in sorted(heads):
            rec = recs.get(f"layer{layer:02d}_head{head:02d}")
            if rec is None:
                continue
            q_abs.append(rec["q_abs_mean"].to(dtype=dtype) if "q_abs_mean" in rec else torch.ones(F, dtype=dtype))
            if "q_mean_real" in rec and "q_mean_imag" in rec:
                q_re.append(rec["q_mean_real"].to(dtype=dtype))
                q_im.append(rec["q_mean_imag"].to(dtype=dtype))
        q_abs_t = torch.stack(q_abs, dim=0)
        if ratio > 1:
            q_abs_t = q_abs_t.reshape(num_kv_heads, ratio, F).mean(dim=1)
        entry = {
            # R-KV files carry no RoPE scaling; the reference falls back to ones when no model config is reachable
            "freq_scale_sq": torch.ones(num_kv_heads, F, device=device, dtype=dtype),
            "q_abs_mean": q_abs_t.to(device),
        }
        if q_re and q_im:
            re_t, im_t = torch.stack(q_re, dim=0), torch.stack(q_im, dim=0)
            if ratio > 1:
                re_t = re_t.reshape(num_kv_heads, ratio, F).mean(dim=1)
                im_t = im_t.reshape(num_kv_heads, ratio, F).mean(dim=1)
            entry["q_mean_complex"] = torch.stack([re_t, im_t], dim=-1).to(device)
        head_stats[layer] = entry
    return metadata, head_stats


def load_frequency_stats(stats_path, device="cpu", dtype: torch.dtype = torch.float32,
                         num_kv_heads: Optional[int] = None) -> Tuple[dict, dict]:
    """(metadata, head_stats) with ``head_stats[layer] = {q_mean_complex [H,F,2], q_abs_mean [H,F], freq_scale_sq [H,F]}``."""
    stats_path = Path(stats_path)
    if not stats_path.exists():
        raise FileNotFoundError(f"Stats file not found: {stats_path}")
    payload = torch.load(stats_path, map_location="cpu", weights_only=False)
    metadata = payload.get("metadata", {})
    recs = payload.get("stats", {})
    if recs and any(_KEY.match(k) for k in recs):
        return _convert_rkv(payload, device, dtype, num_kv_heads)
    missing = [k for k in ("num_attention_heads", "num_kv_heads", "head_dim", "num_layers") if k not in metadata]
    if missing:
        raise ValueError(f"Stats file missing required metadata keys: {missing}. Found keys: {list(metadata.keys())}")
    layer_stats = payload.get("layer_stats", {})
    if not layer_stats:
        raise ValueError("Stats file does not contain 'layer_stats'")
    inv_freq = _inv_freq_from(metadata, int(metadata["head_dim"]) // 2, device)
    if inv_freq is not None:
        metadata["inv_freq"] = inv_freq
    head_stats = {}
    for layer, data in layer_stats.items():
        head_stats[layer] = {k: (v.to(device=device, dtype=dtype) if isinstance(v, torch.Tensor) else v)
                             for k, v in data.items()}
    return metadata, head_stats


def geometric_offsets(offset_max_length: int = 65536, device="cpu") -> torch.Tensor:
    """Scoring offsets 1, 2, 4, ... <= offset_max_length as fp32 (core/compressor.py:222-242)."""
    if int(offset_max_length) < 1:
        raise ValueError(f"offset_max_length must be >= 1, got {offset_max_length}")
    vals, v = [], 1
    while v <= int(offset_max_length):
        vals.append(float(v))
        v *= 2
    return torch.tensor(vals, device=device, dtype=torch.float32)


def resolve_omega(metadata: dict, head_dim: int, device="cpu") -> torch.Tensor:
    """omega = rotary inv_freq: metadata.inv_freq, else rope_theta-based (core/compressor.py:119-194)."""
    inv = metadata.get("inv_freq")
    if isinstance(inv, torch.Tensor):
        return inv.to(device=device, dtype=torch.float32)[: head_dim // 2].contiguous()
    return compute_rope_frequencies(head_dim, float(metadata.get("rope_theta", 10000.0)), device=device)


def resolve_layer_for_stats(layer_idx: int, available_sorted: Sequence[int]) -> int:
    """Layer whose statistics score ``layer_idx``: itself, else wrap modulo the available layers (selector_hf.py:132-143)."""
    if not available_sorted:
        raise RuntimeError("empty_head_stats")
    if layer_idx in available_sorted:
        return layer_idx
    return available_sorted[layer_idx % len(available_sorted)]


def pack_device_stats(head_stats: dict, layer_indices: Sequence[int], omega: torch.Tensor, offsets: torch.Tensor,
                      device, rope_interleaved: bool = False, reduce_to_heads: Optional[int] = None) -> ops.DeviceStats:
    """Stack the statistics of ``layer_indices`` into ``[L, Hs, F]`` fp32 device tensors for the kernels.

    ``reduce_to_heads`` averages each group of statistic heads down to that many heads first
    (selector_hf.py:147-203, used by the legacy per-layer modes).
    """
    avail = tuple(sorted(head_stats.keys()))
    q_re, q_im, q_abs, fs = [], [], [], []
    for l in layer_indices:
        rec = head_stats[resolve_layer_for_stats(int(l), avail)]
        qc = rec["q_mean_complex"].to(torch.float32)
        re_t, im_t = qc[..., 0], qc[..., 1]
        if "q_abs_mean" in rec:
            ab_t = rec["q_abs_mean"].to(torch.float32)
        else:
            ab_t = torch.sqrt(re_t ** 2 + im_t ** 2 + 1e-8)
        fs_t = rec["freq_scale_sq"].to(torch.float32)
        if reduce_to_heads is not None and int(re_t.shape[0]) != reduce_to_heads:
            hs = int(re_t.shape[0])
            if reduce_to_heads <= 0 or hs % reduce_to_heads != 0:
                raise RuntimeError(f"incompatible_head_mapping:source={hs},target={reduce_to_heads}")
            g = hs // reduce_to_heads
            re_t, im_t, ab_t, fs_t = (x.reshape(reduce_to_heads, g, x.shape[-1]).mean(dim=1)
                                      for x in (re_t, im_t, ab_t, fs_t))
        q_re.append(re_t)
        q_im.append(im_t)
        q_abs.append(ab_t)
        fs.append(fs_t)

    def _stack(xs):
        return torch.stack(xs, dim=0).to(device=device, dtype=torch.float32).contiguous()

    return ops.DeviceStats(_stack(q_re), _stack(q_im), _stack(q_abs), _stack(fs),
                           omega.to(device=device, dtype=torch.float32).contiguous(),
                           offsets.to(device=device, dtype=torch.float32).contiguous(), rope_interleaved)
