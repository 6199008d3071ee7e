"""CPU restatement of the reference keep-set selection.  Test infrastructure only.

Follows ``triattention/vllm/runtime/selector_hf.py``: head mapping (:242-275),
raw paged scoring with the GQA expansion (:299-328), streaming z-normalisation
moments (:858-914), guards (:417-441), group max (:277-292), layer mean
(:973-989) and the top-k + ascending sort (:990-1033); the per-layer variants
follow :473-677.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .compaction import gather_request_k_dense, split_kv_axes
from .scoring import score_keys_reference


def streaming_moments(raw: torch.Tensor, chunk_tokens: int = 4096, eps: float = 1e-8):
    """(mean, std_safe) per row of ``raw [Hs, T]`` as the reference accumulates them.

    Chunked fp32 sum and sum of squares, ``var = (sumsq - n*mean^2)/(n-1)``
    clamped at 0, ``std < eps -> 1`` (selector_hf.py:884-913).
    """
    T = int(raw.shape[-1])
    sum_vec = None
    sumsq_vec = None
    start = 0
    while start < T:
        cur = raw[..., start : start + chunk_tokens].to(torch.float32)
        cs = cur.sum(dim=-1)
        cq = (cur * cur).sum(dim=-1)
        sum_vec = cs if sum_vec is None else sum_vec + cs
        sumsq_vec = cq if sumsq_vec is None else sumsq_vec + cq
        start += chunk_tokens
    mean = sum_vec / float(T)
    if T > 1:
        var = (sumsq_vec - float(T) * (mean * mean)) / float(T - 1)
    else:
        var = torch.zeros_like(mean)
    var = torch.clamp(var, min=0.0)
    std = torch.sqrt(var)
    std_safe = torch.where(std < eps, torch.ones_like(std), std)
    return mean, std_safe


def topk_lowest_index(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Ascending indices of the k largest entries per row; equal scores -> lowest index wins.

    The reference uses ``torch.topk(sorted=False)`` then an index sort
    (selector_hf.py:991-1025), which leaves the order among equal scores
    unspecified; this is the deterministic policy the CUDA select implements.
    """
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    keep = order[..., :k]
    return torch.sort(keep, dim=-1).values.contiguous()


def _chunk_tokens(block_size: int, total_tokens: int, score_chunk_max_tokens: int) -> int:
    """selector_hf.py:465-471."""
    upper = max(block_size, int(score_chunk_max_tokens))
    if total_tokens <= upper:
        return max(block_size, total_tokens)
    return upper


def _layer_raw_scores(
    kv_cache: torch.Tensor,
    block_ids: Sequence[int],
    block_size: int,
    total_tokens: int,
    stats_layer: dict,
    omega: torch.Tensor,
    offsets: torch.Tensor,
    round_start: int,
    aggregation: str,
    disable_mlr: bool,
    disable_trig: bool,
    rope_style: str,
    kv_axis: int | None,
):
    """Raw scores ``[Hs, T]`` of one layer, plus (runtime_heads, group_size).

    K is expanded by ``repeat_interleave(group)`` so that query head ``h``
    scores KV head ``h // group`` (selector_hf.py:308-312).
    """
    keys = gather_request_k_dense(kv_cache, block_ids, block_size, total_tokens, kv_axis=kv_axis)  # [1,Hkv,T,D]
    runtime_heads = int(keys.shape[1])
    stats_heads = int(stats_layer["q_mean_real"].shape[0])
    if stats_heads % runtime_heads != 0:
        raise RuntimeError(f"incompatible_head_mapping:source={stats_heads},target={runtime_heads}")
    group = stats_heads // runtime_heads
    expanded = keys.repeat_interleave(group, dim=1) if group > 1 else keys
    raw = score_keys_reference(
        expanded,
        stats_layer["q_mean_real"],
        stats_layer["q_mean_imag"],
        stats_layer["q_abs_mean"],
        stats_layer["freq_scale_sq"],
        omega,
        offsets,
        round_start,
        aggregation=aggregation,
        disable_mlr=disable_mlr,
        disable_trig=disable_trig,
        rope_style=rope_style,
    )[0]
    return raw, runtime_heads, group


def _guard_mask(total_tokens: int, window_size: int, prefill_len: int, protect_prefill: bool):
    """Tokens forced to +inf: the last min(window, T) and, if protected, the prefill (selector_hf.py:417-441)."""
    pos = torch.arange(total_tokens)
    mask = torch.zeros(total_tokens, dtype=torch.bool)
    if window_size > 0:
        recent = min(window_size, total_tokens)
        mask |= pos >= max(0, total_tokens - recent)
    if protect_prefill and prefill_len > 0:
        mask |= pos < prefill_len
    return mask


def final_scores_group_per_head(
    layers: Sequence[tuple],
    stats: dict,
    omega: torch.Tensor,
    offsets: torch.Tensor,
    total_tokens: int,
    round_start: int,
    window_size: int = 128,
    prefill_len: int = 0,
    protect_prefill: bool = False,
    normalize: bool = True,
    aggregation: str = "mean",
    layer_agg: str = "mean",
    disable_mlr: bool = False,
    disable_trig: bool = False,
    rope_style: str = "half",
    score_chunk_max_tokens: int = 4096,
    kv_axis: int | None = None,
    return_raw: bool = False,
):
    """Final per-KV-head scores ``[Hkv, T]`` of the default mode.

    ``layers`` = sequence of ``(layer_idx, kv_cache, block_ids, block_size)``;
    ``stats[layer_idx]`` = dict of ``q_mean_real/q_mean_imag/q_abs_mean/freq_scale_sq [Hs, F]``.
    Order of operations (selector_hf.py:852-989): raw score -> z-norm per
    (layer, query head) over all T -> +inf on guarded tokens -> max over the
    query heads of each KV head -> sum over layers, divided by the layer count
    (or running max when ``layer_agg == 'max'``).
    """
    guard = _guard_mask(total_tokens, window_size, prefill_len, protect_prefill)
    min_bs = min(int(e[3]) for e in layers)
    chunk = _chunk_tokens(min_bs, total_tokens, score_chunk_max_tokens)
    agg = None
    raws = []
    for layer_idx, kv_cache, block_ids, block_size in layers:
        raw, runtime_heads, group = _layer_raw_scores(
            kv_cache, block_ids, block_size, total_tokens, stats[layer_idx], omega, offsets,
            round_start, aggregation, disable_mlr, disable_trig, rope_style, kv_axis,
        )
        if return_raw:
            raws.append(raw)
        z = raw
        if normalize:
            mean, std_safe = streaming_moments(raw, chunk_tokens=chunk)
            z = (raw - mean.view(-1, 1)) / std_safe.view(-1, 1)
        if guard.any():
            z = z.masked_fill(guard.view(1, -1), float("inf"))
        if group > 1:
            z = z.view(runtime_heads, group, -1).max(dim=1).values
        if agg is None:
            agg = z.clone()
        elif layer_agg == "max":
            agg = torch.maximum(agg, z)
        else:
            agg.add_(z)
    final = agg if layer_agg == "max" else agg.div(float(len(layers)))
    if return_raw:
        return final, raws
    return final


def select_group_per_head(layers, stats, omega, offsets, total_tokens, round_start, budget_total, **kw) -> torch.Tensor:
    """Keep indices ``[Hkv, k]`` int64 ascending, k = min(budget, T) (selector_hf.py:749-1033).

    ``T <= budget`` returns the identity keep set (:768-798).
    """
    if total_tokens <= budget_total:
        probe = layers[0][1]
        hkv = int(probe.shape[3])
        return torch.arange(total_tokens, dtype=torch.long).unsqueeze(0).expand(hkv, -1).contiguous()
    final = final_scores_group_per_head(layers, stats, omega, offsets, total_tokens, round_start, **kw)
    k = min(int(budget_total), total_tokens)
    return topk_lowest_index(final, k)


def select_layer_local(
    kv_cache,
    block_ids,
    block_size,
    stats_layer,
    omega,
    offsets,
    total_tokens,
    round_start,
    budget_total,
    mode: str = "per_head",
    group_agg: str = "max",
    reduce_stats: bool = False,
    window_size: int = 128,
    prefill_len: int = 0,
    protect_prefill: bool = False,
    normalize: bool = True,
    aggregation: str = "mean",
    disable_mlr: bool = False,
    disable_trig: bool = False,
    rope_style: str = "half",
    score_chunk_max_tokens: int = 4096,
    kv_axis: int | None = None,
    return_scores: bool = False,
):
    """Per-layer selection (selector_hf.py:473-677): z-norm -> group reduce -> guards -> top-k.

    ``return_scores=True`` returns ``(keep, scores)`` with the rows the top-k ran on (``[Hkv, T]`` or ``[1, T]``).

    ``mode == 'per_head'`` returns ``[Hkv, k]``; ``mode == 'shared'`` takes the
    max over heads first (:636-637) and returns ``[k]``.  ``reduce_stats``
    averages the query-head statistics of each GQA group down to the KV heads
    before scoring (:147-203), which is what the reference does for
    ``legacy_layer_local`` and ``per_layer`` instead of the group max (:251-274).
    """
    if total_tokens <= budget_total:
        return torch.arange(total_tokens, dtype=torch.long)
    if reduce_stats:
        key_cache, _ = split_kv_axes(kv_cache, kv_axis)
        hkv = int(key_cache.shape[2])
        hs = int(stats_layer["q_mean_real"].shape[0])
        if hs != hkv:
            g = hs // hkv
            stats_layer = {k: v.reshape(hkv, g, v.shape[-1]).mean(dim=1).contiguous() for k, v in stats_layer.items()}
    raw, runtime_heads, group = _layer_raw_scores(
        kv_cache, block_ids, block_size, total_tokens, stats_layer, omega, offsets,
        round_start, aggregation, disable_mlr, disable_trig, rope_style, kv_axis,
    )
    z = raw
    if normalize:
        chunk = _chunk_tokens(block_size, total_tokens, score_chunk_max_tokens)
        mean, std_safe = streaming_moments(raw, chunk_tokens=chunk)
        z = (raw - mean.view(-1, 1)) / std_safe.view(-1, 1)
    if group > 1:
        zg = z.view(runtime_heads, group, -1)
        z = zg.mean(dim=1) if group_agg == "mean" else zg.max(dim=1).values
    guard = _guard_mask(total_tokens, window_size, prefill_len, protect_prefill)
    if guard.any():
        z = z.masked_fill(guard.view(1, -1), float("inf"))
    k = min(int(budget_total), total_tokens)
    if mode == "shared":
        z = z.max(dim=0).values
    keep = topk_lowest_index(z, k)
    return (keep, z.view(-1, z.shape[-1])) if return_scores else keep
