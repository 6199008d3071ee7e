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


# ------------------------------------------------------------------------------------------ capture from a model
def find_attention_layers(model) -> list:
    """The ``self_attn`` module of every decoder layer (``model.model.layers[i].self_attn``, scripts/calibrate.py:98-113)."""
    backbone = getattr(model, "model", model)
    layers = getattr(backbone, "layers", None)
    if layers is None:
        raise RuntimeError("Cannot locate transformer layers. Expected model.model.layers.")
    out = []
    for layer in layers:
        attn = getattr(layer, "self_attn", None)
        if attn is None:
            raise RuntimeError("Layer missing self_attn attribute.")
        out.append(attn)
    return out


def _rotate_half(x: torch.Tensor, rope_style: str) -> torch.Tensor:
    if rope_style == "interleaved":
        out = torch.empty_like(x)
        out[..., 0::2] = -x[..., 1::2]
        out[..., 1::2] = x[..., 0::2]
        return out
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def capture_query_stats(model, input_ids: torch.Tensor, rope_style: str = "half", apply_q_norm: bool = False):
    """Statistics of every layer from ONE forward pass of a Hugging Face style decoder (scripts/calibrate.py:116-272).

    A forward pre-hook on each ``self_attn`` recomputes the query projection of the layer's input, rotates it with
    the model's own rotary embedding (positions 0..T-1, times its ``attention_scaling``) and keeps it; after the pass
    the rotation is taken out again and the per-head complex mean and mean magnitude are formed.  ``apply_q_norm``
    additionally applies the module's ``q_norm`` before the rotation (the reference script does not).

    Returns ``(per_layer, info)``: a list of ``{q_mean_real, q_mean_imag, q_abs_mean}`` ``[H, F]`` dictionaries and
    ``{"head_dim", "num_heads", "inv_freq", "attn_scale"}``; feed them to :func:`save_stats`.
    """
    cfg = model.config
    num_heads = int(cfg.num_attention_heads)
    head_dim = int(getattr(cfg, "head_dim", None) or cfg.hidden_size // num_heads)
    attn_layers = find_attention_layers(model)
    backbone = getattr(model, "model", model)
    rotary = backbone.rotary_emb if hasattr(backbone, "rotary_emb") else attn_layers[0].rotary_emb
    attn_scale = float(getattr(rotary, "attention_scaling", 1.0))
    captured: Dict[int, torch.Tensor] = {}

    def tables(q_len: int, device, dtype):
        pos = torch.arange(q_len, device=device).unsqueeze(0)
        return rotary(torch.zeros(1, q_len, head_dim, device=device, dtype=dtype), pos)   # [1, T, D] each

    def make_hook(idx: int):
        def hook(module, args, kwargs):
            hidden = args[0] if args else kwargs.get("hidden_states")
            if hidden is None:
                return
            bsz, q_len, _ = hidden.shape
            q = module.q_proj(hidden).view(bsz, q_len, num_heads, head_dim)
            if apply_q_norm and hasattr(module, "q_norm"):
                q = module.q_norm(q)
            q = q.transpose(1, 2)
            cos, sin = tables(q_len, hidden.device, hidden.dtype)
            captured[idx] = ((q * cos.unsqueeze(1) + _rotate_half(q, rope_style) * sin.unsqueeze(1)) * attn_scale).detach()
        return hook

    handles = [a.register_forward_pre_hook(make_hook(i), with_kwargs=True) for i, a in enumerate(attn_layers)]
    try:
        with torch.no_grad():
            model(input_ids)
    finally:
        for h in handles:
            h.remove()
    T = int(input_ids.shape[1])
    cos_t, sin_t = tables(T, input_ids.device, next(model.parameters()).dtype)
    F = head_dim // 2
    # per-frequency tables [T, F]: the rotary embedding repeats (half) or interleaves its F angles over D; the
    # reference divides the attention scaling out of cos/sin before inverting (scripts/calibrate.py:75-95)
    sel = slice(0, None, 2) if rope_style == "interleaved" else slice(0, F)
    cos_f = (cos_t[0, :, sel] / attn_scale).float()
    sin_f = (sin_t[0, :, sel] / attn_scale).float()
    per_layer = []
    for i in range(len(attn_layers)):
        if i not in captured:
            raise RuntimeError(f"no queries captured for layer {i}")
        per_layer.append(query_frequency_stats(captured.pop(i).float(), cos_f, sin_f, attn_scale, rope_style))
    inv_freq = getattr(rotary, "inv_freq", None)
    info = {"head_dim": head_dim, "num_heads": num_heads, "attn_scale": attn_scale,
            "inv_freq": inv_freq.detach().float().cpu() if isinstance(inv_freq, torch.Tensor) else None}
    return per_layer, info
