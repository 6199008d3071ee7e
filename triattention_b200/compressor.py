"""Dense-tensor API of the reference (core/scoring.py ``compute_scores``, core/compressor.py
``TriAttentionCompressor``) on top of the paged kernels.

Dense K ``[B, H, T, D]`` is repacked into a paged buffer in which every KV head is its own "layer" (own base
pointer, own rows of statistics) and every batch entry its own "request"; the scorer kernel then runs unchanged.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _native, ops
from .config import TriAttentionConfig
from .rope import resolve_rope_spec
from .stats import geometric_offsets, load_frequency_stats, resolve_omega

_BS = 16


def _dense_as_paged(key_states: torch.Tensor):
    """K [B, H, T, D] -> (view with L=H "layers", block table [B, nblk], buffer)."""
    B, H, T, D = key_states.shape
    nblk = (T + _BS - 1) // _BS
    buf = torch.zeros((H, B * nblk * _BS, D), dtype=torch.bfloat16, device=key_states.device)
    buf.view(H, B, nblk * _BS, D)[:, :, :T] = key_states.permute(1, 0, 2, 3).to(torch.bfloat16)
    ptrs = torch.tensor([buf[h].data_ptr() for h in range(H)], dtype=torch.int64, device=buf.device)
    view = ops.PagedCacheView(k_ptrs=ptrs, v_ptrs=ptrs, num_layers=H, num_blocks=B * nblk, block_size=_BS,
                              num_kv_heads=1, head_dim=D, block_stride=_BS * D, token_stride=D, head_stride=D,
                              device=buf.device, dtype=buf.dtype)
    bt = torch.arange(B * nblk, dtype=torch.int32, device=buf.device).view(B, nblk)
    return view, bt, buf


def _raw_scores_dense(key_states: torch.Tensor, q_re, q_im, q_abs, fs, omega, offsets, round_start: int,
                      aggregation: str, disable_mlr: bool, disable_trig: bool, rope_style: str):
    """(raw [H, B, 1, t_pad, gp], moments, layout, seq_lens) for dense K and statistics ``[Hs, F]``, Hs = H*g."""
    B, H, T, D = key_states.shape
    dev = key_states.device
    Hs = int(q_re.shape[0])
    if Hs % H != 0:
        raise RuntimeError(f"incompatible_head_mapping:source={Hs},target={H}")
    g = Hs // H
    F = D // 2

    def _prep(x):
        return x.to(device=dev, dtype=torch.float32).reshape(H, g, F).contiguous()

    dstats = ops.DeviceStats(_prep(q_re), _prep(q_im), _prep(q_abs), _prep(fs),
                             omega.to(device=dev, dtype=torch.float32).contiguous(),
                             offsets.to(device=dev, dtype=torch.float32).contiguous(), rope_style == "interleaved")
    view, bt, _buf = _dense_as_paged(key_states)
    layout = view.layout(B, g, int(bt.shape[1]), rope_interleaved=dstats.rope_interleaved)
    seq = torch.full((B,), T, dtype=torch.int32, device=dev)
    rs = torch.full((B,), int(round_start), dtype=torch.int32, device=dev)
    agg = _native.OFFSETS_MAX if aggregation == "max" else _native.OFFSETS_MEAN
    flags = (_native.FLAG_DISABLE_MLR if disable_mlr else 0) | (_native.FLAG_DISABLE_TRIG if disable_trig else 0)
    w = ops.prep_weights(dstats, rs, agg, flags)
    raw, mom = ops.score_paged(view, layout, bt, seq, w, agg, int(offsets.numel()))
    return raw, mom, layout, seq, g


def compute_scores(key_states: torch.Tensor, cache_positions: Optional[torch.Tensor], head_stats: Dict[str, torch.Tensor],
                   omega: torch.Tensor, offsets: torch.Tensor, freq_scale_sq: torch.Tensor, config: TriAttentionConfig,
                   round_start: Optional[int] = None, trig_cache=None) -> torch.Tensor:
    """Raw importance scores ``[B, Hs, T]`` fp32 (``[B, T]`` head-mean in per_layer mode) - core/scoring.py:18-76.

    ``head_stats`` = {'q_mean_complex' [Hs, F, 2], optional 'q_abs_mean' [Hs, F]}; when Hs is a multiple of the
    number of KV heads H, query head h scores KV head h // (Hs/H).
    """
    if not key_states.is_cuda:
        raise _native.NativeLibraryError(
            f"{_native.TRITON_SCORING_REQUIRED_MARKER}:tensor_not_on_cuda:key_states (there is no CPU path)")
    B, H, T, D = key_states.shape
    qc = head_stats["q_mean_complex"]
    q_re, q_im = qc[..., 0], qc[..., 1]
    q_abs = head_stats["q_abs_mean"] if "q_abs_mean" in head_stats else torch.sqrt(q_re ** 2 + q_im ** 2 + 1e-8)
    if round_start is None:
        round_start = int(cache_positions.max().item()) if cache_positions is not None else T - 1
    raw, _mom, _layout, _seq, g = _raw_scores_dense(
        key_states, q_re, q_im, q_abs, freq_scale_sq, omega, offsets, int(round_start), config.score_aggregation,
        config.disable_mlr, config.disable_trig, config.rope_style)
    # raw [H, B, 1, t_pad, gp] -> [B, H*g, T]
    scores = raw[:, :, 0, :T, :g].permute(1, 0, 3, 2).reshape(B, H * g, T)
    if config.pruning_mode == "per_layer":
        scores = scores.mean(dim=1)
    return scores.to(dtype=config.topk_dtype)


class TriAttentionCompressor:
    """Statistics + RoPE frequencies + offsets, and the dense batch-1 ``compress`` (core/compressor.py:27-346)."""

    def __init__(self, config: TriAttentionConfig):
        self.config = config
        self.metadata: Optional[dict] = None
        self.head_stats: Optional[dict] = None
        self.inv_freq: Optional[torch.Tensor] = None
        self.omega: Optional[torch.Tensor] = None
        self.freq_scale_sq: Optional[torch.Tensor] = None
        self.offsets: Optional[torch.Tensor] = None
        self.absolute_position = 0
        self.compression_count = 0
        self._initialized = False

    def _lazy_init(self) -> None:
        if self._initialized:
            return
        cfg = self.config
        if cfg.stats_path is None:
            raise ValueError("stats_path must be specified in TriAttentionConfig.")
        self.metadata, self.head_stats = load_frequency_stats(cfg.stats_path, device=cfg.device, dtype=torch.float32,
                                                              num_kv_heads=cfg.num_kv_heads)
        cfg.head_dim = cfg.head_dim or int(self.metadata["head_dim"])
        cfg.num_kv_heads = cfg.num_kv_heads or int(self.metadata["num_kv_heads"])
        cfg.num_layers = cfg.num_layers or int(self.metadata["num_layers"])
        if "rope_style" in self.metadata:
            cfg.rope_style = str(self.metadata["rope_style"])
        # metadata.inv_freq, then a local model config under model_path, then metadata rope_theta (default 1e4)
        spec = resolve_rope_spec(self.metadata, cfg.head_dim, model_path=cfg.model_path)
        self.inv_freq = (spec.inv_freq.to(cfg.device) if spec is not None
                         else resolve_omega(self.metadata, cfg.head_dim, device=cfg.device))
        self.omega = self.inv_freq
        F = cfg.head_dim // 2
        self.freq_scale_sq = torch.zeros(cfg.num_layers, cfg.num_kv_heads, F, device=cfg.device, dtype=torch.float32)
        for layer in range(cfg.num_layers):
            rec = self.head_stats.get(layer)
            if rec is not None and "freq_scale_sq" in rec:
                self.freq_scale_sq[layer] = rec["freq_scale_sq"]
        self.offsets = geometric_offsets(cfg.offset_max_length, device=cfg.device)
        self._initialized = True

    def reset(self) -> None:
        self.absolute_position = 0
        self.compression_count = 0

    def compress(self, key_states: torch.Tensor, value_states: torch.Tensor,
                 cache_positions: Optional[torch.Tensor] = None, layer_idx: int = 0
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(K, V, keep indices) with at most ``kv_budget`` tokens per head; indices ascending per head.

        Compression fires when the cache holds at least ``kv_budget + divide_length`` tokens
        (core/state.py:82-125); otherwise the inputs come back unchanged with identity indices.
        """
        self._lazy_init()
        cfg = self.config
        B, H, T, D = key_states.shape
        if B > 1:
            raise ValueError(f"TriAttention currently only supports batch_size=1 for compression. Got batch_size={B}.")
        self.absolute_position = max(self.absolute_position, T)
        if T < cfg.kv_budget + cfg.divide_length:
            return key_states, value_states, torch.arange(T, device=key_states.device)
        if layer_idx not in self.head_stats:
            raise ValueError(f"No stats found for layer {layer_idx}")
        rec = self.head_stats[layer_idx]
        qc = rec["q_mean_complex"]
        q_re, q_im = qc[..., 0], qc[..., 1]
        q_abs = rec["q_abs_mean"] if "q_abs_mean" in rec else torch.sqrt(q_re ** 2 + q_im ** 2 + 1e-8)
        raw, mom, layout, seq, _g = _raw_scores_dense(
            key_states, q_re, q_im, q_abs, self.freq_scale_sq[layer_idx], self.omega, self.offsets,
            self.absolute_position, cfg.score_aggregation, cfg.disable_mlr, cfg.disable_trig, cfg.rope_style)
        # per (head-as-layer) scores: z-norm, window guard, no layer reduction -> [H, 1, 1, t_pad]
        fin = ops.finalize_scores(layout, raw, mom, seq, None, cfg.window_size, cfg.sparse_normalize_scores,
                                  _native.REDUCE_MAX, _native.REDUCE_NONE, _native.REDUCE_NONE)
        k = min(cfg.kv_budget, T)
        kc = torch.tensor([k], dtype=torch.int32, device=key_states.device)
        rows = fin.view(-1, fin.shape[-1])
        if cfg.pruning_mode == "per_layer":
            raise NotImplementedError("dense per_layer compression is served by the runtime selector (shared mode)")
        keep = ops.select_topk(rows, seq, kc, 1, int(rows.shape[0]), k).long()  # [H, k]
        idx = keep.unsqueeze(0).unsqueeze(-1).expand(1, H, k, D)
        out_k = torch.gather(key_states, 2, idx)
        out_v = torch.gather(value_states, 2, idx)
        self.compression_count += 1
        return out_k, out_v, keep.unsqueeze(0)
