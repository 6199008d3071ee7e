"""Configuration of the runtime hook and of the scoring algorithm.

``TriAttentionRuntimeConfig`` keeps the environment contract of the reference
(runtime/config.py:19-276): the same ``TRIATTN_RUNTIME_*`` names, defaults and
validation messages.  ``require_triton_scoring`` is read as "require the
native scorer"; there is no non-native scorer here, so it only controls
whether configuration errors raise or return a status string.
``TriAttentionConfig`` mirrors the algorithm dataclass of core/config.py:13-206.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Optional

import torch

_TRUE = {"1", "true", "yes", "on"}
_FALSE = {"0", "false", "no", "off"}


def _parse_bool(raw: str) -> bool:
    value = raw.strip().lower()
    if value in _TRUE:
        return True
    if value in _FALSE:
        return False
    raise ValueError(f"Invalid boolean value: {raw!r}")


def _parse_path(raw: str) -> Optional[Path]:
    raw = raw.strip()
    return Path(raw) if raw else None


# legacy variable -> runtime variable (plugin.py:37-45)
_LEGACY_ENV = {
    "TRIATTENTION_KV_BUDGET": "TRIATTN_RUNTIME_KV_BUDGET",
    "TRIATTENTION_DIVIDE_LENGTH": "TRIATTN_RUNTIME_DIVIDE_LENGTH",
    "TRIATTENTION_WINDOW_SIZE": "TRIATTN_RUNTIME_WINDOW_SIZE",
    "TRIATTENTION_LOG_DECISIONS": "TRIATTN_RUNTIME_LOG_DECISIONS",
    "TRIATTENTION_STATS_PATH": "TRIATTN_RUNTIME_SPARSE_STATS_PATH",
}
# switches the plugin turns on unless the operator set them (plugin.py:47-51)
_STRICT_DEFAULTS = ("ENABLE_EXPERIMENTAL_KV_COMPACTION", "ENABLE_EXPERIMENTAL_BLOCK_RECLAIM",
                    "REQUIRE_TRITON_SCORING", "REQUIRE_PHYSICAL_RECLAIM")


def bridge_legacy_env(environ=None) -> None:
    """Map the older ``TRIATTENTION_*`` variables onto ``TRIATTN_RUNTIME_*`` (plugin.py:37-58).

    A runtime variable that is already set (non-empty) wins; empty legacy values are ignored; the four strictness
    switches default to ``true``; ``TRIATTENTION_PRUNING_MODE`` is lower-cased and its old spelling
    ``per_layer_head`` becomes ``per_layer_per_head``.  Call before :meth:`TriAttentionRuntimeConfig.from_env`.
    """
    env = os.environ if environ is None else environ
    for legacy, runtime in _LEGACY_ENV.items():
        value = env.get(legacy)
        if not env.get(runtime) and value:
            env[runtime] = value
    for name in _STRICT_DEFAULTS:
        env.setdefault("TRIATTN_RUNTIME_" + name, "true")
    if not env.get("TRIATTN_RUNTIME_PRUNING_MODE"):
        mode = (env.get("TRIATTENTION_PRUNING_MODE") or "").strip().lower()
        if mode:
            env["TRIATTN_RUNTIME_PRUNING_MODE"] = "per_layer_per_head" if mode == "per_layer_head" else mode


@dataclass
class TriAttentionRuntimeConfig:
    """Runtime config loaded by scheduler and worker (fields and defaults of runtime/config.py:27-60)."""

    kv_budget: int = 2048
    divide_length: int = 128
    protect_prefill: bool = False
    disable_compression: bool = False
    enable_kv_usage_trigger: bool = False
    kv_usage_trigger: float = 0.98
    kv_usage_release: float = 0.90
    enable_experimental_kv_compaction: bool = True
    enable_experimental_block_reclaim: bool = True
    require_triton_scoring: bool = True
    require_physical_reclaim: bool = True
    log_decisions: bool = True
    fail_on_effective_len_regression: bool = True
    effective_len_regression_ratio: float = 0.9
    effective_len_guard_divide_multiples: int = 2
    score_chunk_max_tokens: int = 4096
    sparse_stats_path: Optional[Path] = None
    model_path: Optional[Path] = None
    pruning_mode: str = "per_head"
    sparse_score_aggregation: str = "mean"
    sparse_normalize_scores: bool = True
    window_size: int = 128
    include_prefill_in_budget: bool = True
    per_head_selection_semantics: str = "hf_aligned_global_per_head"
    layer_perhead_aggregation: str = "max"
    per_layer_aggregation: str = "max"
    allow_per_layer_mode: bool = False
    disable_mlr: bool = False
    disable_trig: bool = False
    disable_top_n_high_freq: int = 0
    # additions of this implementation (not read by the reference)
    preserve_dropped_tokens: bool = False
    """Also rewrite the dropped tokens behind the kept prefix (whole-region byte equality with the reference)."""
    use_cuda_graph: bool = False
    """Replay the fused step from a CUDA graph once a geometry repeats (steady-state decode compressions)."""

    @classmethod
    def from_env(cls, prefix: str = "TRIATTN_RUNTIME_") -> "TriAttentionRuntimeConfig":
        """Read every field from ``<prefix><FIELD_NAME_UPPER>``; unset variables keep the default."""
        kwargs = {}
        for f in fields(cls):
            raw = os.environ.get(prefix + f.name.upper())
            if raw is None:
                continue
            default = f.default
            if isinstance(default, bool):
                kwargs[f.name] = _parse_bool(raw)
            elif isinstance(default, int):
                kwargs[f.name] = int(raw)
            elif isinstance(default, float):
                kwargs[f.name] = float(raw)
            elif f.name in ("sparse_stats_path", "model_path"):
                kwargs[f.name] = _parse_path(raw)
            else:
                stripped = raw.strip()
                if stripped:
                    kwargs[f.name] = stripped
        config = cls(**kwargs)
        config.validate()
        return config

    def validate(self) -> None:
        if self.kv_budget <= 0:
            raise ValueError(f"kv_budget must be > 0, got {self.kv_budget}")
        if self.divide_length <= 0:
            raise ValueError(f"divide_length must be > 0, got {self.divide_length}")
        if not (0.0 < self.kv_usage_trigger <= 1.0):
            raise ValueError(f"kv_usage_trigger must be in (0, 1], got {self.kv_usage_trigger}")
        if not (0.0 <= self.kv_usage_release <= 1.0):
            raise ValueError(f"kv_usage_release must be in [0, 1], got {self.kv_usage_release}")
        if self.kv_usage_release > self.kv_usage_trigger:
            raise ValueError("kv_usage_release should be <= kv_usage_trigger to avoid hysteresis inversion")
        if self.pruning_mode not in {"per_layer", "per_head", "per_layer_per_head"}:
            raise ValueError(
                "pruning_mode must be one of {'per_layer','per_head','per_layer_per_head'}, "
                f"got {self.pruning_mode!r}")
        if self.pruning_mode == "per_layer" and not self.allow_per_layer_mode:
            raise ValueError(
                "pruning_mode='per_layer' is disabled by default in the runtime to prevent accidental use. "
                "Set allow_per_layer_mode=True (env TRIATTN_RUNTIME_ALLOW_PER_LAYER_MODE=1) for explicit opt-in.")
        if self.sparse_score_aggregation not in {"mean", "max"}:
            raise ValueError(f"sparse_score_aggregation must be 'mean' or 'max', got {self.sparse_score_aggregation!r}")
        if self.per_head_selection_semantics not in {"legacy_layer_local", "hf_aligned_global_per_head"}:
            raise ValueError(
                "per_head_selection_semantics must be one of {'legacy_layer_local','hf_aligned_global_per_head'}, "
                f"got {self.per_head_selection_semantics!r}")
        if self.layer_perhead_aggregation not in {"max", "mean"}:
            raise ValueError(f"layer_perhead_aggregation must be 'max' or 'mean', got {self.layer_perhead_aggregation!r}")
        if self.per_layer_aggregation not in {"max", "mean", "pure_mean"}:
            raise ValueError(
                f"per_layer_aggregation must be one of {{'max','mean','pure_mean'}}, got {self.per_layer_aggregation!r}")
        if self.window_size < 0:
            raise ValueError(f"window_size must be >= 0, got {self.window_size}")
        if self.disable_top_n_high_freq < 0:
            raise ValueError(f"disable_top_n_high_freq must be >= 0, got {self.disable_top_n_high_freq}")
        if not (0.0 < self.effective_len_regression_ratio <= 1.0):
            raise ValueError(
                f"effective_len_regression_ratio must be in (0, 1], got {self.effective_len_regression_ratio}")
        if self.effective_len_guard_divide_multiples < 1:
            raise ValueError(
                f"effective_len_guard_divide_multiples must be >= 1, got {self.effective_len_guard_divide_multiples}")
        if self.score_chunk_max_tokens < 1:
            raise ValueError(f"score_chunk_max_tokens must be >= 1, got {self.score_chunk_max_tokens}")
        if (self.enable_experimental_kv_compaction and self.require_physical_reclaim
                and not self.enable_experimental_block_reclaim):
            raise ValueError(
                "enable_experimental_kv_compaction requires enable_experimental_block_reclaim=True when "
                "require_physical_reclaim=True")


@dataclass
class TriAttentionConfig:
    """Algorithm parameters of the dense compressor API (core/config.py:13-206)."""

    kv_budget: int = 2048
    divide_length: int = 128
    sparse_round_window: int = 32
    pruning_mode: str = "per_head"
    score_aggregation: str = "mean"
    offset_max_length: int = 65536
    disable_top_n_high_freq: int = 0
    disable_mlr: bool = False
    disable_trig: bool = False
    include_prefill_in_budget: bool = True
    protect_prefill: bool = True
    window_size: int = 128
    sparse_normalize_scores: bool = True
    topk_dtype: torch.dtype = torch.float32
    compute_dtype: torch.dtype = torch.bfloat16
    device: torch.device = field(default_factory=lambda: torch.device("cuda"))
    stats_path: Optional[Path] = None
    model_path: Optional[Path] = None
    rope_style: str = "half"
    head_dim: Optional[int] = None
    num_kv_heads: Optional[int] = None
    num_layers: Optional[int] = None
    seed: Optional[int] = None
    enable_debug_logging: bool = False

    def __post_init__(self):
        if isinstance(self.stats_path, str):
            self.stats_path = Path(self.stats_path)
        if isinstance(self.model_path, str):
            self.model_path = Path(self.model_path)
        if self.kv_budget <= 0:
            raise ValueError(f"kv_budget must be positive, got {self.kv_budget}")
        if self.divide_length <= 0:
            raise ValueError(f"divide_length must be positive, got {self.divide_length}")
        if self.window_size < 0:
            raise ValueError(f"window_size cannot be negative, got {self.window_size}")
        if self.window_size >= self.kv_budget:
            raise ValueError(f"window_size ({self.window_size}) must be less than kv_budget ({self.kv_budget})")
        if self.pruning_mode == "per_layer_per_head":
            self.pruning_mode = "per_head"
        if self.score_aggregation not in {"mean", "max"}:
            raise ValueError(f"Unsupported score_aggregation: {self.score_aggregation}")
