"""Rotary frequencies of the served model, resolved on the host without any network access.

The scorer needs the model's own ``inv_freq`` (omega) and the square of the factor its rotary embedding
multiplies cos/sin with (``freq_scale_sq``).  The reference finds them, in this order, in the statistics
metadata (``inv_freq``), in the model config it fetches by name (core/utils.py:186-297,
core/compressor.py:119-194 via common/rope_utils.py:30-90), and finally falls back to a plain
``rope_theta`` (default 10000) - silently, so a Qwen3 or Llama-3 statistics file that carries neither key
is scored with the wrong frequencies when the Hub is unreachable.

Here the model config comes from what the worker already holds: a local ``config.json`` under
``config.model_path`` (or the runner's model path when that is a directory), the runner's
``model_config.hf_config`` / ``hf_text_config`` object, or the ``rope_theta`` / ``rope_scaling`` entries that
newer statistics files carry in their metadata.  The frequency formulas are the published ones (plain RoPE,
linear position interpolation, the Llama-3.1 wavelength-band rescaling, YaRN's NTK-by-parts ramp with its
``0.1 ln(s) + 1`` attention factor).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Optional

import torch


@dataclass(frozen=True)
class RopeSpec:
    """inv_freq ``[head_dim/2]`` fp32 and the factor applied to cos/sin (1 for unscaled rotary embeddings)."""

    inv_freq: torch.Tensor
    attention_factor: float
    source: str


def _plain(head_dim: int, theta: float) -> torch.Tensor:
    idx = torch.arange(0, head_dim, 2, dtype=torch.int64).to(torch.float32)
    return 1.0 / (float(theta) ** (idx / float(head_dim)))


def _llama3(inv_freq: torch.Tensor, p: Mapping[str, Any]) -> torch.Tensor:
    factor = float(p["factor"])
    low, high = float(p["low_freq_factor"]), float(p["high_freq_factor"])
    old_ctx = float(p["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv_freq
    scaled = torch.where(wavelen > old_ctx / low, inv_freq / factor, inv_freq)
    smooth = (old_ctx / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * scaled / factor + smooth * scaled
    medium = (~(wavelen < old_ctx / high)) & (~(wavelen > old_ctx / low))
    return torch.where(medium, blended, scaled)


def _yarn(head_dim: int, theta: float, p: Mapping[str, Any], max_position: Optional[int]):
    old_ctx = float(p["original_max_position_embeddings"])
    factor = p.get("factor")
    if factor is None:
        if not max_position:
            raise ValueError("yarn scaling without 'factor' needs max_position_embeddings")
        factor = float(max_position) / old_ctx
    factor = float(factor)

    def mscale(scale: float, m: float = 1.0) -> float:
        return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0

    attention_factor = p.get("attention_factor")
    if attention_factor is None:
        m, m_all = p.get("mscale"), p.get("mscale_all_dim")
        attention_factor = mscale(factor, m) / mscale(factor, m_all) if (m and m_all) else mscale(factor)
    beta_fast = float(p.get("beta_fast") or 32)
    beta_slow = float(p.get("beta_slow") or 1)

    def correction_dim(rotations: float) -> float:
        return head_dim * math.log(old_ctx / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))

    lo, hi = correction_dim(beta_fast), correction_dim(beta_slow)
    if p.get("truncate", True):
        lo, hi = math.floor(lo), math.ceil(hi)
    lo, hi = max(lo, 0), min(hi, head_dim - 1)
    if lo == hi:
        hi += 0.001
    ramp = torch.clamp((torch.arange(head_dim // 2, dtype=torch.float32) - lo) / (hi - lo), 0, 1)
    pos_freqs = float(theta) ** (torch.arange(0, head_dim, 2).to(torch.float32) / head_dim)
    extrapolation, interpolation = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)
    keep = 1.0 - ramp
    return interpolation * (1.0 - keep) + extrapolation * keep, float(attention_factor)


def rope_spec_from_parameters(head_dim: int, rope_theta: float, rope_scaling: Optional[Mapping[str, Any]] = None,
                              max_position_embeddings: Optional[int] = None, source: str = "parameters") -> RopeSpec:
    """RopeSpec from ``rope_theta`` and a ``rope_scaling`` / ``rope_parameters`` dictionary (None = plain RoPE)."""
    if head_dim <= 0 or head_dim % 2:
        raise ValueError(f"head_dim must be a positive even number, got {head_dim}")
    p = dict(rope_scaling or {})
    kind = str(p.get("rope_type", p.get("type", "default")) or "default").lower()
    theta = float(p.get("rope_theta", rope_theta))
    inv = _plain(head_dim, theta)
    af = 1.0
    if kind in ("default", "dynamic", "none"):   # dynamic NTK only changes beyond the trained length
        pass
    elif kind == "linear":
        inv = inv / float(p["factor"])
    elif kind == "llama3":
        inv = _llama3(inv, p)
    elif kind == "yarn":
        inv, af = _yarn(head_dim, theta, p, max_position_embeddings)
    else:
        raise ValueError(f"unsupported rope scaling type {kind!r}")
    return RopeSpec(inv.to(torch.float32).contiguous(), float(af), source)


def _get(cfg: Any, name: str, default=None):
    if isinstance(cfg, Mapping):
        return cfg.get(name, default)
    return getattr(cfg, name, default)


def rope_spec_from_model_config(cfg: Any, head_dim: Optional[int] = None, source: str = "model_config") -> Optional[RopeSpec]:
    """RopeSpec from a Hugging Face style config: a ``config.json`` dictionary or a config object.

    Understands both spellings: ``rope_theta`` + ``rope_scaling`` and the newer ``rope_parameters`` dictionary that
    carries ``rope_theta`` itself.  Returns None when the config names no ``rope_theta`` at all.
    """
    if cfg is None:
        return None
    text = _get(cfg, "text_config")
    if text is not None and _get(cfg, "rope_theta") is None and _get(cfg, "rope_parameters") is None:
        cfg = text
    params = _get(cfg, "rope_parameters")
    scaling = params if isinstance(params, Mapping) else _get(cfg, "rope_scaling")
    theta = _get(cfg, "rope_theta")
    if theta is None and isinstance(scaling, Mapping):
        theta = scaling.get("rope_theta")
    if theta is None:
        return None
    hd = _get(cfg, "head_dim")
    if hd is None:
        hidden, heads = _get(cfg, "hidden_size"), _get(cfg, "num_attention_heads")
        hd = int(hidden) // int(heads) if hidden and heads else head_dim
    if hd is None:
        return None
    partial = _get(cfg, "partial_rotary_factor")
    if partial is None and isinstance(scaling, Mapping):
        partial = scaling.get("partial_rotary_factor")
    rot_dim = int(int(hd) * float(partial)) if partial else int(hd)
    spec = rope_spec_from_parameters(rot_dim, float(theta), scaling if isinstance(scaling, Mapping) else None,
                                     _get(cfg, "max_position_embeddings"), source)
    if head_dim is not None and spec.inv_freq.numel() < head_dim // 2:
        return None
    return spec


def _local_config_json(path: Any) -> Optional[dict]:
    try:
        p = Path(str(path)).expanduser()
    except Exception:
        return None
    f = p / "config.json" if p.is_dir() else (p if p.name == "config.json" and p.is_file() else None)
    if f is None or not f.is_file():
        return None
    try:
        return json.loads(f.read_text())
    except Exception:
        return None


def resolve_rope_spec(metadata: Mapping[str, Any], head_dim: int, model_path: Any = None,
                      base_runner: Any = None) -> Optional[RopeSpec]:
    """Frequencies for scoring, or None when nothing names them (the caller decides whether that is fatal).

    Order: ``metadata['inv_freq']``; a local ``config.json`` under ``model_path`` or the runner's model path; the
    runner's in-memory model config; ``rope_theta`` (+ ``rope_scaling``) written into the statistics metadata.
    """
    F = head_dim // 2
    inv = metadata.get("inv_freq")
    if isinstance(inv, (list, tuple)):
        inv = torch.tensor(inv, dtype=torch.float32)
    if isinstance(inv, torch.Tensor):
        if inv.numel() < F:
            raise ValueError(f"metadata.inv_freq has fewer elements than required by head_dim={head_dim}: "
                             f"got {inv.numel()}, expected at least {F}")
        return RopeSpec(inv.detach().to("cpu", torch.float32)[:F].contiguous(), 1.0, "metadata.inv_freq")

    model_cfgs = []
    for owner in (base_runner, getattr(base_runner, "vllm_config", None)):
        mc = getattr(owner, "model_config", None) if owner is not None else None
        if mc is not None:
            model_cfgs.append(mc)
    paths = [model_path] + [getattr(mc, "model", None) for mc in model_cfgs]
    for path in paths:
        if path is None:
            continue
        cfg = _local_config_json(path)
        spec = rope_spec_from_model_config(cfg, head_dim, f"config.json:{path}") if cfg else None
        if spec is not None:
            return spec
    for mc in model_cfgs:
        for attr in ("hf_text_config", "hf_config"):
            spec = rope_spec_from_model_config(getattr(mc, attr, None), head_dim, f"runner.model_config.{attr}")
            if spec is not None:
                return spec

    raw = metadata.get("rkv_metadata") if isinstance(metadata.get("rkv_metadata"), Mapping) else metadata
    if raw.get("rope_theta") is not None:
        return rope_spec_from_parameters(head_dim, float(raw["rope_theta"]), raw.get("rope_scaling"),
                                         raw.get("max_position_embeddings"), "metadata.rope_theta")
    return None
