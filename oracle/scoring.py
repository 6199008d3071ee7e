"""CPU restatement of the reference key scorer.  Test infrastructure only.

Follows ``triattention/vllm/core/scoring.py:255-362`` (``compute_scores_pytorch``)
with K upcast to fp32 before any arithmetic (the reference's GPU kernel casts
in-kernel, ``triattention/vllm/core/kernels/triton_scoring.py:263-264``), and
``triattention/vllm/core/compressor.py:222-242`` for the offset set.
"""
from __future__ import annotations

import numpy as np
import torch


def geometric_offsets(offset_max_length: int = 65536) -> torch.Tensor:
    """Offsets 1, 2, 4, ... <= offset_max_length as fp32 (compressor.py:228-242)."""
    if offset_max_length < 1:
        raise ValueError(f"offset_max_length must be >= 1, got {offset_max_length}")
    vals = []
    v = 1
    while v <= int(offset_max_length):
        vals.append(float(v))
        v *= 2
    return torch.tensor(vals, dtype=torch.float32)


def _split_complex(key_states: torch.Tensor, rope_style: str):
    """K -> (real, imag) halves per RoPE layout (scoring.py:275-282)."""
    D = key_states.shape[-1]
    F = D // 2
    if rope_style == "interleaved":
        pairs = key_states.reshape(*key_states.shape[:-1], F, 2)
        return pairs[..., 0], pairs[..., 1]
    return key_states[..., :F], key_states[..., F:]


def score_keys_reference(
    key_states: torch.Tensor,
    q_mean_real: torch.Tensor,
    q_mean_imag: torch.Tensor,
    q_abs_mean: torch.Tensor,
    freq_scale_sq: torch.Tensor,
    omega: torch.Tensor,
    offsets: torch.Tensor,
    round_start: int,
    aggregation: str = "mean",
    disable_mlr: bool = False,
    disable_trig: bool = False,
    rope_style: str = "half",
) -> torch.Tensor:
    """Raw scores ``[B, H, T]`` fp32 for keys ``[B, H, T, D]`` and stats ``[H, F]``.

    Same operation order as scoring.py:264-356: per offset ``t = round_start +
    offset`` (a Python float times an fp32 tensor, so the phase is rounded to
    fp32, :313,:322), ``sum_f fs*(Re*cos - Im*sin)`` (:325-332), mean or max
    over offsets (:336-339), then the magnitude term with
    ``|q_mean| = sqrt(qr^2+qi^2+1e-8)`` (:264) and ``|k| = sqrt(kr^2+ki^2)`` (:283).
    """
    k = key_states.to(torch.float32)
    qr = q_mean_real.to(torch.float32)
    qi = q_mean_imag.to(torch.float32)
    qa = q_abs_mean.to(torch.float32)
    fs = freq_scale_sq.to(torch.float32)
    omega = omega.to(torch.float32)
    k_real, k_imag = _split_complex(k, rope_style)
    q_mean_abs = torch.sqrt(qr ** 2 + qi ** 2 + 1e-8)
    k_abs = torch.sqrt(k_real ** 2 + k_imag ** 2)
    qr_e = qr.unsqueeze(0).unsqueeze(2)
    qi_e = qi.unsqueeze(0).unsqueeze(2)
    prod_real = qr_e * k_real + qi_e * k_imag
    prod_imag = qi_e * k_real - qr_e * k_imag
    fs_e = fs.unsqueeze(0).unsqueeze(2)
    om_e = omega.view(1, 1, 1, -1)
    per_offset = []
    for off in offsets:
        t = round_start + off.item()
        if not disable_trig:
            phase = t * om_e
            term = fs_e * (prod_real * torch.cos(phase) - prod_imag * torch.sin(phase))
        else:
            term = torch.zeros_like(prod_real)
        per_offset.append(term.sum(dim=-1))
    stacked = torch.stack(per_offset, dim=0)
    if aggregation == "mean":
        scores = stacked.mean(dim=0)
    elif aggregation == "max":
        scores = stacked.max(dim=0).values
    else:
        raise ValueError(f"Unsupported score_aggregation: {aggregation}")
    coef = qa if disable_mlr else (qa - q_mean_abs)
    extra = (k_abs * coef.unsqueeze(0).unsqueeze(2) * fs_e).sum(dim=-1)
    return scores + extra


def score_keys_exact64(
    key_states: torch.Tensor,
    q_mean_real: torch.Tensor,
    q_mean_imag: torch.Tensor,
    q_abs_mean: torch.Tensor,
    freq_scale_sq: torch.Tensor,
    omega: torch.Tensor,
    offsets: torch.Tensor,
    round_start: int,
    aggregation: str = "mean",
    disable_mlr: bool = False,
    disable_trig: bool = False,
    rope_style: str = "half",
) -> np.ndarray:
    """The same formula in float64 (numpy) with the reference's fp32-rounded phases.

    Used for error budgeting: how far the fp32 reference and the CUDA kernel
    each sit from exact arithmetic on identical inputs.
    """
    k = key_states.to(torch.float32).numpy().astype(np.float64)
    qr = q_mean_real.to(torch.float32).numpy().astype(np.float64)[None, :, None, :]
    qi = q_mean_imag.to(torch.float32).numpy().astype(np.float64)[None, :, None, :]
    qa = q_abs_mean.to(torch.float32).numpy().astype(np.float64)[None, :, None, :]
    fs = freq_scale_sq.to(torch.float32).numpy().astype(np.float64)[None, :, None, :]
    om32 = omega.to(torch.float32).numpy()
    D = k.shape[-1]
    F = D // 2
    if rope_style == "interleaved":
        kr, ki = k[..., 0::2], k[..., 1::2]
    else:
        kr, ki = k[..., :F], k[..., F:]
    pr = qr * kr + qi * ki
    pi = qi * kr - qr * ki
    per = []
    for off in offsets.tolist():
        t32 = np.float32(float(round_start) + float(off))
        phase32 = (t32 * om32).astype(np.float32)  # fp32-rounded phase is part of the contract
        ph = phase32.astype(np.float64)
        if disable_trig:
            per.append(np.zeros(pr.shape[:-1]))
        else:
            per.append((fs * (pr * np.cos(ph) - pi * np.sin(ph))).sum(-1))
    st = np.stack(per, 0)
    base = st.mean(0) if aggregation == "mean" else st.max(0)
    q_mean_abs = np.sqrt(qr ** 2 + qi ** 2 + 1e-8)
    coef = qa if disable_mlr else (qa - q_mean_abs)
    extra = (np.sqrt(kr ** 2 + ki ** 2) * coef * fs).sum(-1)
    return base + extra
