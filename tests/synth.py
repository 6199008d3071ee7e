"""Seeded synthetic inputs for the score -> select -> compact path.

Stands in for real serving traces: Qwen3-/Llama-shaped paged bf16 KV caches and
calibrated Q-centre statistics with the value distributions the benchmark
configurations name.  Everything is generated on the CPU from a seeded
``torch.Generator`` so that the CPU checker and the CUDA kernels see
bit-identical inputs; tensors are moved to the device by the caller.

Stats layout follows the reference's on-disk "R-KV" format
(scripts/calibrate.py:231-271, triattention/vllm/core/utils.py:57-70).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch


def seed_for(config_idx: int, sweep_idx: int = 0, rank: int = 0) -> int:
    """Seed convention: 20260000 + 1000*config + 10*sweep + rank."""
    return 20260000 + 1000 * int(config_idx) + 10 * int(sweep_idx) + int(rank)


def rope_inv_freq(head_dim: int, theta: float, llama3: Optional[dict] = None) -> torch.Tensor:
    """RoPE inverse frequencies ``theta^(-2f/head_dim)`` as fp32 ``[head_dim/2]``.

    ``llama3`` = {"factor", "low_freq_factor", "high_freq_factor",
    "original_max_position_embeddings"} applies the published Llama-3.1
    frequency rescaling (wavelength-dependent division by ``factor`` with a
    smooth band in between).
    """
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
    inv_freq = 1.0 / (float(theta) ** (idx / float(head_dim)))
    if llama3 is None:
        return inv_freq.contiguous()
    factor = float(llama3["factor"])
    low = float(llama3["low_freq_factor"])
    high = float(llama3["high_freq_factor"])
    old_ctx = float(llama3["original_max_position_embeddings"])
    low_wavelen = old_ctx / low
    high_wavelen = old_ctx / high
    wavelen = 2.0 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_ctx / wavelen - low) / (high - low)
    smoothed = (1.0 - smooth) * scaled / factor + smooth * scaled
    is_medium = (~(wavelen < high_wavelen)) & (~(wavelen > low_wavelen))
    return torch.where(is_medium, smoothed, scaled).to(torch.float32).contiguous()


@dataclass
class SyntheticStats:
    """Per (layer, query head, frequency) Q-centre statistics, fp32."""

    q_mean_real: torch.Tensor  # [L, Hq, F]
    q_mean_imag: torch.Tensor  # [L, Hq, F]
    q_abs_mean: torch.Tensor   # [L, Hq, F]
    inv_freq: torch.Tensor     # [F]
    head_dim: int
    rope_style: str = "half"

    @property
    def num_layers(self) -> int:
        return int(self.q_mean_real.shape[0])

    @property
    def num_heads(self) -> int:
        return int(self.q_mean_real.shape[1])


def make_stats(
    num_layers: int,
    num_q_heads: int,
    head_dim: int,
    inv_freq: torch.Tensor,
    gen: torch.Generator,
    rope_style: str = "half",
) -> SyntheticStats:
    """Centre magnitude log-uniform in [0.1, 5], phase U[0, 2pi), mean |q| = magnitude * U[1, 1.5]."""
    F = head_dim // 2
    shape = (num_layers, num_q_heads, F)
    lo, hi = math.log(0.1), math.log(5.0)
    mag = torch.exp(lo + (hi - lo) * torch.rand(shape, generator=gen, dtype=torch.float32))
    phase = 2.0 * math.pi * torch.rand(shape, generator=gen, dtype=torch.float32)
    ratio = 1.0 + 0.5 * torch.rand(shape, generator=gen, dtype=torch.float32)
    return SyntheticStats(
        q_mean_real=(mag * torch.cos(phase)).contiguous(),
        q_mean_imag=(mag * torch.sin(phase)).contiguous(),
        q_abs_mean=(mag * ratio).contiguous(),
        inv_freq=inv_freq.to(torch.float32).contiguous(),
        head_dim=head_dim,
        rope_style=rope_style,
    )


def save_stats_pt(stats: SyntheticStats, path: Path, extra_metadata: Optional[dict] = None) -> None:
    """Write ``stats`` in the reference's R-KV ``.pt`` format with ``inv_freq`` in the metadata."""
    L, H = stats.num_layers, stats.num_heads
    payload_stats = {}
    sampled = []
    for l in range(L):
        for h in range(H):
            payload_stats[f"layer{l:02d}_head{h:02d}"] = {
                "q_mean_real": stats.q_mean_real[l, h].clone(),
                "q_mean_imag": stats.q_mean_imag[l, h].clone(),
                "q_abs_mean": stats.q_abs_mean[l, h].clone(),
            }
            sampled.append([l, h])
    metadata = {
        "head_dim": int(stats.head_dim),
        "rope_style": stats.rope_style,
        "sampled_heads": sampled,
        "inv_freq": stats.inv_freq.clone(),
    }
    if extra_metadata:
        metadata.update(extra_metadata)
    torch.save({"metadata": metadata, "stats": payload_stats}, str(path))


def make_rotated_keys(
    num_kv_heads: int,
    num_tokens: int,
    head_dim: int,
    inv_freq: torch.Tensor,
    gen: torch.Generator,
    start_position: int = 0,
    rope_style: str = "half",
    positions: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Post-RoPE K for one (layer, request): bf16 ``[T, Hkv, D]`` (token-major, as a paged block stores it).

    Pre-RoPE channels are N(0,1) times a per-(head, channel) scale drawn
    log-uniform in [0.1, 10] (outlier bands), rotated at positions
    ``start_position .. start_position+T-1`` (or ``positions``).
    """
    F = head_dim // 2
    lo, hi = math.log(0.1), math.log(10.0)
    scale = torch.exp(lo + (hi - lo) * torch.rand((num_kv_heads, head_dim), generator=gen, dtype=torch.float32))
    pre = torch.randn((num_tokens, num_kv_heads, head_dim), generator=gen, dtype=torch.float32) * scale
    if positions is None:
        positions = torch.arange(start_position, start_position + num_tokens, dtype=torch.float32)
    ang = positions.to(torch.float32).view(-1, 1, 1) * inv_freq.to(torch.float32).view(1, 1, F)
    c, s = torch.cos(ang), torch.sin(ang)
    if rope_style == "interleaved":
        pr, pi = pre[..., 0::2], pre[..., 1::2]
    else:
        pr, pi = pre[..., :F], pre[..., F:]
    rr = pr * c - pi * s
    ri = pr * s + pi * c
    if rope_style == "interleaved":
        out = torch.stack([rr, ri], dim=-1).reshape(num_tokens, num_kv_heads, head_dim)
    else:
        out = torch.cat([rr, ri], dim=-1)
    return out.to(torch.bfloat16).contiguous()


def make_values(num_kv_heads: int, num_tokens: int, head_dim: int, gen: torch.Generator) -> torch.Tensor:
    """V ~ N(0,1), bf16 ``[T, Hkv, D]``."""
    return torch.randn((num_tokens, num_kv_heads, head_dim), generator=gen, dtype=torch.float32).to(torch.bfloat16)


def random_block_ids(num_needed: int, num_blocks_total: int, gen: torch.Generator, first_free: int = 0) -> list[int]:
    """``num_needed`` distinct block ids drawn as a random permutation of ``[first_free, num_blocks_total)``."""
    perm = torch.randperm(num_blocks_total - first_free, generator=gen)[:num_needed] + first_free
    return [int(x) for x in perm.tolist()]


def write_tokens_to_paged(
    kv_cache: torch.Tensor,
    kv_axis: int,
    block_ids: list[int],
    block_size: int,
    keys_thd: torch.Tensor,
    values_thd: torch.Tensor,
) -> None:
    """Scatter token-major ``[T, H, D]`` K/V into a 5-D paged cache (K/V axis 0 or 1)."""
    T = int(keys_thd.shape[0])
    if kv_axis == 0:
        kc, vc = kv_cache[0], kv_cache[1]
    else:
        kc, vc = kv_cache[:, 0], kv_cache[:, 1]
    tok = torch.arange(T)
    blk = torch.as_tensor(block_ids, dtype=torch.long)[tok // block_size]
    off = tok % block_size
    kc[blk, off] = keys_thd.to(kc.dtype)
    vc[blk, off] = values_thd.to(vc.dtype)


def make_paged_layer(
    num_blocks_total: int,
    block_size: int,
    num_kv_heads: int,
    head_dim: int,
    kv_axis: int = 0,
    dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Zero paged cache for one layer: ``[2, nb, bs, H, D]`` (kv_axis 0) or ``[nb, 2, bs, H, D]`` (kv_axis 1)."""
    if kv_axis == 0:
        return torch.zeros((2, num_blocks_total, block_size, num_kv_heads, head_dim), dtype=dtype)
    return torch.zeros((num_blocks_total, 2, block_size, num_kv_heads, head_dim), dtype=dtype)
