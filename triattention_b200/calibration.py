"""Producer of the frequency-statistics file the scorer consumes (reference: scripts/calibrate.py:49-272).

The reference hooks a Hugging Face model, captures the rotated queries of one forward pass per layer, removes the
rotary embedding again and stores, per (layer, query head, frequency), the complex mean of the un-rotated query and
the mean of its magnitude.  Running a model is outside this package; what is here is the arithmetic on captured
queries and the on-disk format, so that statistics can be produced from any source of rotated queries
(an engine hook, a trace) without the reference script.  Offline, host-side torch code: not on the hot path.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

import torch


def rotary_tables(inv_freq: torch.Tensor, num_positions: int, start: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of ``position * inv_freq`` as fp32 ``[num_positions, F]``."""
    pos = torch.arange(start, start + num_positions, dtype=torch.float32, device=inv_freq.device)
    ang = pos[:, None] * inv_freq.to(torch.float32)[None, :]
    return torch.cos(ang), torch.sin(ang)


def as_complex_pairs(x: torch.Tensor, rope_style: str = "half") -> torch.Tensor:
    """``[..., D]`` real -> ``[..., D/2]`` complex: (x[f], x[f + D/2]) for "half", (x[2f], x[2f+1]) for "interleaved"."""
    xf = x.to(torch.float32) if x.dtype in (torch.bfloat16, torch.float16) else x
    if rope_style == "interleaved":
        return torch.complex(xf[..., 0::2].contiguous(), xf[..., 1::2].contiguous())
    F = xf.shape[-1] // 2
    return torch.complex(xf[..., :F].contiguous(), xf[..., F:].contiguous())


def unrotate_queries(q_rot: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, attn_scale: float = 1.0,
                     rope_style: str = "half") -> torch.Tensor:
    """Complex un-rotated queries ``[..., T, F]`` from rotated ``q_rot [..., T, D]`` and per-frequency tables ``[T, F]``.

    A rotary embedding multiplies the complex pair of frequency f by ``exp(i * pos * w_f)`` (and the reference
    scales by ``attn_scale``); the inverse multiplies by the conjugate and divides by the scale.
    """
    if attn_scale == 0:
        raise ValueError("attention scaling factor must be non-zero")
    z = as_complex_pairs(q_rot, rope_style) / attn_scale
    return z * torch.complex(cos.to(z.real.dtype), -sin.to(z.real.dtype))


def query_frequency_stats(q_rot: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, attn_scale: float = 1.0,
                          rope_style: str = "half") -> Dict[str, torch.Tensor]:
    """Statistics of one layer from rotated queries ``[H, T, D]``: ``q_mean_real``, ``q_mean_imag``, ``q_abs_mean`` ``[H, F]``."""
    if q_rot.ndim == 4:
        if q_rot.shape[0] != 1:
            raise ValueError("calibration uses a single trace: expected a leading batch dimension of 1")
        q_rot = q_rot[0]
    base = unrotate_queries(q_rot, cos, sin, attn_scale, rope_style)  # [H, T, F] complex
    mean = base.mean(dim=1)
    return {"q_mean_real": mean.real.contiguous(), "q_mean_imag": mean.imag.contiguous(),
            "q_abs_mean": base.abs().mean(dim=1).contiguous()}


def stats_payload(per_layer: Iterable[Dict[str, torch.Tensor]], head_dim: int, rope_style: str = "half",
                  inv_freq: Optional[torch.Tensor] = None, extra_metadata: Optional[dict] = None) -> dict:
    """The ``{"metadata", "stats"}`` dictionary of the statistics file (keys ``layerLL_headHH``)."""
    stats, sampled = {}, []
    for l, layer in enumerate(per_layer):
        H = int(layer["q_mean_real"].shape[0])
        for h in range(H):
            stats[f"layer{l:02d}_head{h:02d}"] = {k: layer[k][h].detach().cpu() for k in
                                                   ("q_mean_real", "q_mean_imag", "q_abs_mean")}
            sampled.append([l, h])
    meta = {"num_traces": 1, "head_dim": int(head_dim), "rope_style": rope_style, "sampled_heads": sampled}
    if inv_freq is not None:
        meta["inv_freq"] = inv_freq.detach().cpu().to(torch.float32)
    if extra_metadata:
        meta.update(extra_metadata)
    return {"metadata": meta, "stats": stats}


def save_stats(path, per_layer: Iterable[Dict[str, torch.Tensor]], head_dim: int, rope_style: str = "half",
               inv_freq: Optional[torch.Tensor] = None, extra_metadata: Optional[dict] = None) -> None:
    out = Path(path)
    out.parent.mkdir(parents=True, exist_ok=True)
    torch.save(stats_payload(per_layer, head_dim, rope_style, inv_freq, extra_metadata), out)
