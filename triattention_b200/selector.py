"""Keep-set selector with the interface of the reference's ``build_triattention_selector``
(runtime/selector_hf.py:15-1083), running on the CUDA kernels.

The returned callables take the same keyword arguments and return the same result dicts
(``{"mode": "per_head"|"shared", "indices": int64 tensor ascending, ...}``).  Scoring, z-normalisation,
guards, group/layer reductions and top-k all happen on the device; the reference's 4096-token chunking
(:465-471) has no counterpart because the scorer streams the paged cache and nothing is materialised.
"""
from __future__ import annotations

import os
import warnings
from pathlib import Path
from typing import Any, Callable, Iterable, Optional

import torch

from . import _native, ops
from .config import TriAttentionRuntimeConfig
from .constants import TRITON_SCORING_REQUIRED_MARKER
from .kv_compaction import kv_axis_hint
from .rope import resolve_rope_spec, rope_spec_from_parameters
from .stats import geometric_offsets, load_frequency_stats, pack_device_stats


def _dense_keys_view(keys_dense: torch.Tensor, block_size: int = 16):
    """Repack dense K ``[1, H, T, D]`` as a one-layer paged K buffer ``[nb, bs, H, D]`` (consecutive blocks)."""
    if keys_dense.ndim != 4 or int(keys_dense.shape[0]) != 1:
        raise ValueError(f"keys_dense must be [1, H, T, D], got {tuple(keys_dense.shape)}")
    _, H, T, D = keys_dense.shape
    nb = (T + block_size - 1) // block_size
    buf = torch.zeros((nb * block_size, H, D), dtype=torch.bfloat16, device=keys_dense.device)
    buf[:T] = keys_dense[0].transpose(0, 1).to(torch.bfloat16)
    buf = buf.view(nb, block_size, H, D)
    ptr = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=buf.device)
    view = ops.PagedCacheView(k_ptrs=ptr, v_ptrs=ptr, num_layers=1, num_blocks=nb, block_size=block_size,
                              num_kv_heads=H, head_dim=D, block_stride=buf.stride(0), token_stride=buf.stride(1),
                              head_stride=buf.stride(2), device=buf.device, dtype=buf.dtype)
    return view, list(range(nb)), buf


class FusedCompactionError(RuntimeError):
    """The compaction stage of the fused group call failed (scoring and selection were fine)."""


def load_scoring_state(stats_path, config, base_runner: Any | None, strict: bool) -> dict:
    """Statistics of ``stats_path`` plus the frequencies they are scored with (host side, no device work).

    omega and the cos/sin factor of the model's rotary embedding come from the statistics metadata, else from the
    model config the worker holds locally (the reference fetches that config by model name: core/compressor.py:119-194,
    core/utils.py:186-297).  When nothing names them: fatal in strict mode, a warning and ``rope_theta = 10000``
    (core/compressor.py:186-191) otherwise.
    """
    metadata, head_stats = load_frequency_stats(stats_path, device="cpu", dtype=torch.float32)
    head_dim = int(metadata["head_dim"])
    spec = resolve_rope_spec(metadata, head_dim, model_path=getattr(config, "model_path", None),
                             base_runner=base_runner)
    if spec is None:
        if strict:
            raise RuntimeError(
                f"{TRITON_SCORING_REQUIRED_MARKER}:rope_unresolved:stats metadata has no inv_freq/rope_theta "
                "and no local model config was found (set TRIATTN_RUNTIME_MODEL_PATH to the model directory)")
        warnings.warn("TriAttention: rotary frequencies unresolved, falling back to rope_theta=10000; "
                      "keep sets will be wrong for models with another base or scaled RoPE")
        spec = rope_spec_from_parameters(head_dim, float(metadata.get("rope_theta", 10000.0)),
                                         source="fallback.rope_theta")
    if spec.attention_factor != 1.0 and "rkv_metadata" in metadata:
        # converted calibration files carry freq_scale_sq = 1; the reference replaces it with the square of the
        # rotary embedding's cos/sin factor when it can build the model's rotary (core/utils.py:253-297)
        for rec in head_stats.values():
            rec["freq_scale_sq"] = rec["freq_scale_sq"] * float(spec.attention_factor) ** 2
    return dict(loaded=True, metadata=metadata, head_stats=head_stats, head_dim=head_dim, omega=spec.inv_freq,
                rope_source=spec.source, attention_factor=spec.attention_factor, offsets=geometric_offsets(65536),
                interleaved=str(metadata.get("rope_style", "half")) == "interleaved")


def build_triattention_selector(
    config: TriAttentionRuntimeConfig,
    base_runner: Any | None = None,
) -> tuple[Optional[Callable[..., Any]], Optional[Callable[..., Any]], str]:
    """(select_keep_indices, select_keep_indices_for_group, status) - see selector_hf.py:15-22."""
    requested_mode = config.pruning_mode
    if requested_mode == "per_layer" and not bool(getattr(config, "allow_per_layer_mode", False)):
        raise RuntimeError(
            f"{TRITON_SCORING_REQUIRED_MARKER}:per_layer_mode_disabled:set allow_per_layer_mode=True for explicit opt-in")
    strict = bool(config.enable_experimental_kv_compaction and config.require_triton_scoring)
    if config.sparse_stats_path is None:
        if strict:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:stats_path_not_set")
        return None, None, "stats_path_not_set"
    stats_path = Path(config.sparse_stats_path).expanduser()
    if not stats_path.exists():
        if strict:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:stats_path_not_found")
        return None, None, "stats_path_not_found"
    try:
        _native.load()
    except Exception as exc:
        raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:import_failed:{type(exc).__name__}") from exc
    if requested_mode not in {"per_layer", "per_head", "per_layer_per_head"}:
        if strict:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:unsupported_pruning_mode:{requested_mode}")
        return None, None, f"unsupported_pruning_mode:{requested_mode}"
    semantics = config.per_head_selection_semantics
    offset_agg = _native.OFFSETS_MAX if config.sparse_score_aggregation == "max" else _native.OFFSETS_MEAN
    flags = (_native.FLAG_DISABLE_MLR if config.disable_mlr else 0) | (_native.FLAG_DISABLE_TRIG if config.disable_trig else 0)

    state: dict = {"loaded": False}
    packed_cache: dict = {}

    def _load():
        if not state["loaded"]:
            state.update(load_scoring_state(stats_path, config, base_runner, strict))
        return state

    _load()  # at start-up: a statistics file whose frequencies cannot be resolved must not fail mid-serving

    def _packed(layer_indices, device, reduce_to: Optional[int]) -> ops.DeviceStats:
        st = _load()
        key = (tuple(int(x) for x in layer_indices), str(device), reduce_to)
        hit = packed_cache.get(key)
        if hit is None:
            hit = pack_device_stats(st["head_stats"], layer_indices, st["omega"], st["offsets"], device,
                                    rope_interleaved=st["interleaved"], reduce_to_heads=reduce_to)
            packed_cache[key] = hit
        return hit

    def _recent(total_tokens: int) -> int:
        if total_tokens <= 0 or config.window_size <= 0:
            return 0
        return min(config.window_size, total_tokens)

    def _group_of(stats_heads: int, runtime_heads: int) -> int:
        if runtime_heads <= 0 or stats_heads % runtime_heads != 0:
            raise RuntimeError(
                f"{TRITON_SCORING_REQUIRED_MARKER}:incompatible_head_mapping:source={stats_heads},target={runtime_heads}")
        return stats_heads // runtime_heads

    def _score_and_select(view: ops.PagedCacheView, block_ids, layer_indices, total_tokens: int, prefill_len: int,
                          protect_prefill: bool, round_start: int, k: int, *, reduce_stats: bool, group_reduce: int,
                          head_reduce: int, layer_reduce: int) -> torch.Tensor:
        """keep rows ``[Lo*Ho, k]`` int64 for one request."""
        dev = view.device
        try:
            dstats = _packed(layer_indices, dev, view.num_kv_heads if reduce_stats else None)
            g = _group_of(dstats.num_heads, view.num_kv_heads)
            if isinstance(block_ids, torch.Tensor):
                bt = block_ids.to(device=dev, dtype=torch.int32).reshape(1, -1).contiguous()
            else:
                bt = torch.as_tensor([int(x) for x in block_ids], dtype=torch.int32, device=dev).reshape(1, -1)
            need = (total_tokens + view.block_size - 1) // view.block_size
            if need > int(bt.shape[1]):
                raise IndexError(f"token range requires block_idx={need - 1}, but only {int(bt.shape[1])} blocks exist")
            bt = bt[:, :need].contiguous()
            layout = view.layout(1, g, need, rope_interleaved=dstats.rope_interleaved)
            meta = torch.tensor([total_tokens, int(round_start), k, int(prefill_len), 0], dtype=torch.int32, device=dev)
            seq, rs, kc, pre, status = meta[0:1], meta[1:2], meta[2:3], meta[3:4], meta[4:5]
            w = ops.prep_weights(dstats, rs, offset_agg, flags)
            raw, mom = ops.score_paged(view, layout, bt, seq, w, offset_agg, int(dstats.offsets.numel()), status)
            fin = ops.finalize_scores(layout, raw, mom, seq, pre if (protect_prefill and prefill_len > 0) else None,
                                      _recent(total_tokens), bool(config.sparse_normalize_scores), group_reduce,
                                      head_reduce, layer_reduce)
            rows = fin.view(-1, fin.shape[-1])
            keep = ops.select_topk(rows, seq, kc, 1, int(rows.shape[0]), k, status)
            bits = int(status.item())
            if bits:
                raise _native.NativeLibraryError(f"device_status:{bits}")
        except _native.NativeLibraryError as exc:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:score_failed:{type(exc).__name__}") from exc
        return keep.long()

    def _select_keep_indices(*, keys_dense: torch.Tensor | None = None, kv_cache: torch.Tensor | None = None,
                             block_ids=None, block_size: int | None = None, total_tokens: int, prefill_len: int,
                             protect_prefill: bool, layer_idx: int, round_start: int, budget_total: int):
        """Per-layer selection (selector_hf.py:679-747)."""
        if total_tokens <= budget_total:
            return {"mode": "shared", "indices": list(range(total_tokens))}
        if protect_prefill and config.include_prefill_in_budget and prefill_len > budget_total:
            return None
        if keys_dense is not None:
            view, block_ids, _keep_alive = _dense_keys_view(keys_dense)
        elif kv_cache is not None and block_ids is not None and block_size is not None:
            view = ops.PagedCacheView.from_layers([kv_cache], kv_axis=kv_axis_hint(kv_cache))
        else:
            raise RuntimeError("missing scoring inputs for selector")
        k = min(int(budget_total), int(total_tokens))
        if k <= 0:
            return {"mode": "shared", "indices": []}
        hf_group = ((requested_mode == "per_head" and semantics == "hf_aligned_global_per_head")
                    or requested_mode == "per_layer_per_head")
        group_reduce = _native.REDUCE_MAX
        if requested_mode == "per_layer_per_head" and config.layer_perhead_aggregation == "mean":
            group_reduce = _native.REDUCE_MEAN
        shared = requested_mode == "per_layer"
        keep = _score_and_select(
            view, block_ids, [layer_idx], total_tokens, prefill_len, protect_prefill, round_start, k,
            reduce_stats=not hf_group, group_reduce=group_reduce,
            head_reduce=_native.REDUCE_MAX if shared else _native.REDUCE_NONE, layer_reduce=_native.REDUCE_NONE)
        if shared:
            return {"mode": "shared", "indices": keep[0].contiguous()}
        return {"mode": "per_head", "indices": keep.contiguous()}

    def _select_keep_indices_for_group_per_head(
        *, layer_inputs: list | None = None, layer_input_iter: Callable[[], Iterable] | None = None,
        layer_kv_iter: Callable[[], Iterable] | None = None, total_tokens: int, prefill_len: int,
        protect_prefill: bool, round_start: int, budget_total: int,
    ):
        """One keep set per KV head shared by all layers of the group (selector_hf.py:749-1083)."""
        if requested_mode != "per_head" or semantics != "hf_aligned_global_per_head":
            return None
        if layer_kv_iter is not None:
            entries = list(layer_kv_iter())
            mode = "paged"
        elif layer_input_iter is not None:
            entries = list(layer_input_iter())
            mode = "dense"
        else:
            entries = list(layer_inputs or [])
            mode = "dense"
        if total_tokens <= budget_total:
            if not entries:
                return {"mode": "per_head", "indices": []}
            first = entries[0][1]
            heads = int(first.shape[3]) if mode == "paged" else int(first.shape[1])
            ident = torch.arange(total_tokens, dtype=torch.long, device=first.device)
            return {"mode": "per_head", "indices": ident.unsqueeze(0).expand(heads, -1).contiguous()}
        if protect_prefill and config.include_prefill_in_budget and prefill_len > budget_total:
            return None
        if not entries:
            return None
        k = min(int(budget_total), int(total_tokens))
        if k <= 0:
            return {"mode": "per_head", "indices": []}
        layer_indices = [int(e[0]) for e in entries]
        if mode == "paged":
            agg = os.environ.get("TRIATTN_RUNTIME_DEBUG_GROUP_PERHEAD_AGG_MODE", "mean").strip().lower()
            if agg not in {"mean", "max"}:
                agg = "mean"
            caches = [e[1] for e in entries]
            block_ids = entries[0][2]
            view = ops.PagedCacheView.from_layers(caches, kv_axis=kv_axis_hint(caches[0]))
            keep = _score_and_select(
                view, block_ids, layer_indices, total_tokens, prefill_len, protect_prefill, round_start, k,
                reduce_stats=False, group_reduce=_native.REDUCE_MAX, head_reduce=_native.REDUCE_NONE,
                layer_reduce=_native.REDUCE_MAX if agg == "max" else _native.REDUCE_MEAN)
        else:
            agg = "mean"
            # dense inputs: repack every layer into one paged K buffer set (one view per layer, same block ids)
            views = [_dense_keys_view(e[1]) for e in entries]
            v0 = views[0][0]
            ptrs = torch.cat([v[0].k_ptrs for v in views])
            view = ops.PagedCacheView(k_ptrs=ptrs, v_ptrs=ptrs, num_layers=len(views), num_blocks=v0.num_blocks,
                                      block_size=v0.block_size, num_kv_heads=v0.num_kv_heads, head_dim=v0.head_dim,
                                      block_stride=v0.block_stride, token_stride=v0.token_stride,
                                      head_stride=v0.head_stride, device=v0.device, dtype=v0.dtype)
            keep = _score_and_select(
                view, views[0][1], layer_indices, total_tokens, prefill_len, protect_prefill, round_start, k,
                reduce_stats=False, group_reduce=_native.REDUCE_MAX, head_reduce=_native.REDUCE_NONE,
                layer_reduce=_native.REDUCE_MEAN)
        return {
            "mode": "per_head",
            "indices": keep.contiguous(),
            "semantic": "hf_aligned_global_per_head",
            "group_agg_mode": agg,
            "debug_group_layer_indices": layer_indices,
            "debug_recent_count": _recent(total_tokens),
        }

    fused_engines: dict = {}

    def _compress_group_fused(*, caches: list, layer_indices: list, block_ids, total_tokens: int, prefill_len: int,
                              protect_prefill: bool, round_start: int, budget_total: int):
        """Default mode in ONE native call: score -> select -> compact every layer of the group with the shared
        per-KV-head keep set (what the group selector followed by the per-layer compaction loop produce,
        selector_hf.py:749-1083 + layout_engine.py:112-139).  Returns the selector's result dictionary (plus
        ``cache_len_after``) or None when this request needs the staged path (another mode, nothing to drop,
        protected prefill larger than the budget)."""
        if requested_mode != "per_head" or semantics != "hf_aligned_global_per_head":
            return None
        if total_tokens <= budget_total or not caches:
            return None
        if protect_prefill and config.include_prefill_in_budget and prefill_len > budget_total:
            return None
        k = min(int(budget_total), int(total_tokens))
        if k <= 0:
            return None
        from . import engine as _engine
        agg = os.environ.get("TRIATTN_RUNTIME_DEBUG_GROUP_PERHEAD_AGG_MODE", "mean").strip().lower()
        if agg not in {"mean", "max"}:
            agg = "mean"
        try:
            view = ops.PagedCacheView.from_layers(caches, kv_axis=kv_axis_hint(caches[0]))
            dstats = _packed([int(i) for i in layer_indices], view.device, None)
            _group_of(dstats.num_heads, view.num_kv_heads)
            comp = fused_engines.get(str(view.device))
            if comp is None:
                comp = _engine.PagedCompressor(dstats, use_cuda_graph=bool(getattr(config, "use_cuda_graph", False)))
                fused_engines[str(view.device)] = comp
            comp.stats = dstats
            comp.window = int(config.window_size) if config.window_size > 0 else 0
            comp.normalize = bool(config.sparse_normalize_scores)
            comp.offset_agg, comp.flags = offset_agg, flags
            comp.layer_reduce = _native.REDUCE_MAX if agg == "max" else _native.REDUCE_MEAN
            ids = block_ids.tolist() if isinstance(block_ids, torch.Tensor) else [int(x) for x in block_ids]
            res = comp.compress(view, [ids], [int(total_tokens)], [int(round_start)], [k],
                                prefill_lens=[int(prefill_len)] if (protect_prefill and prefill_len > 0) else None)
            if res.device_status & ~_native.DEV_BAD_KEEP_INDEX:
                raise _native.NativeLibraryError(f"device_status:{res.device_status}")
        except _native.NativeLibraryError as exc:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:score_failed:{type(exc).__name__}") from exc
        if res.device_status:
            # only the compaction stage reports keep-index faults: a soft failure, as in the per-layer loop
            raise FusedCompactionError(f"device_status:{res.device_status}")
        return {
            "mode": "per_head",
            # the engine's own int32 output buffer, valid until its next call: the hook only needs the row count
            # here (the cache is already compacted); callers that keep the indices must copy them
            "indices": res.keep[0],
            "semantic": "hf_aligned_global_per_head",
            "group_agg_mode": agg,
            "debug_group_layer_indices": [int(i) for i in layer_indices],
            "debug_recent_count": _recent(total_tokens),
            "cache_len_after": k,
        }

    def _compress_group_fused_batch(*, caches: list, layer_indices: list, items: list) -> list:
        """The fused default-mode step for SEVERAL requests of one KV-cache group in one native call.

        ``items`` holds, per request, the keyword arguments of :func:`_compress_group_fused` other than ``caches``
        and ``layer_indices``.  Returns one entry per item: the selector's result dictionary, or None for a request
        that needs the staged path (same rules as the single-request form).  Results equal those of calling the
        single-request form request after request: the scorer's moments and the top-k do not depend on the batch.
        """
        out: list = [None] * len(items)
        if requested_mode != "per_head" or semantics != "hf_aligned_global_per_head" or not caches:
            return out
        todo = []
        for n, it in enumerate(items):
            total, budget = int(it["total_tokens"]), int(it["budget_total"])
            if total <= budget:
                continue
            if it["protect_prefill"] and config.include_prefill_in_budget and int(it["prefill_len"]) > budget:
                continue
            k = min(budget, total)
            if k > 0:
                todo.append((n, k))
        if not todo:
            return out
        from . import engine as _engine
        agg = os.environ.get("TRIATTN_RUNTIME_DEBUG_GROUP_PERHEAD_AGG_MODE", "mean").strip().lower()
        if agg not in {"mean", "max"}:
            agg = "mean"
        try:
            view = ops.PagedCacheView.from_layers(caches, kv_axis=kv_axis_hint(caches[0]))
            dstats = _packed([int(i) for i in layer_indices], view.device, None)
            _group_of(dstats.num_heads, view.num_kv_heads)
            comp = fused_engines.get(str(view.device))
            if comp is None:
                comp = _engine.PagedCompressor(dstats, use_cuda_graph=bool(getattr(config, "use_cuda_graph", False)))
                fused_engines[str(view.device)] = comp
            comp.stats = dstats
            comp.window = int(config.window_size) if config.window_size > 0 else 0
            comp.normalize = bool(config.sparse_normalize_scores)
            comp.offset_agg, comp.flags = offset_agg, flags
            comp.layer_reduce = _native.REDUCE_MAX if agg == "max" else _native.REDUCE_MEAN
            ids, totals, starts, ks, prefill = [], [], [], [], []
            for n, k in todo:
                it = items[n]
                b = it["block_ids"]
                ids.append(b.tolist() if isinstance(b, torch.Tensor) else [int(x) for x in b])
                totals.append(int(it["total_tokens"]))
                starts.append(int(it["round_start"]))
                ks.append(k)
                prefill.append(int(it["prefill_len"]) if (it["protect_prefill"] and int(it["prefill_len"]) > 0) else 0)
            res = comp.compress(view, ids, totals, starts, ks, prefill_lens=prefill if any(prefill) else None)
            if res.device_status & ~_native.DEV_BAD_KEEP_INDEX:
                raise _native.NativeLibraryError(f"device_status:{res.device_status}")
        except _native.NativeLibraryError as exc:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:score_failed:{type(exc).__name__}") from exc
        if res.device_status:
            raise FusedCompactionError(f"device_status:{res.device_status}")
        for row, (n, k) in enumerate(todo):
            out[n] = {
                "mode": "per_head",
                "indices": res.keep[row][:, :k],  # a view of the engine's buffer, valid until its next call
                "semantic": "hf_aligned_global_per_head",
                "group_agg_mode": agg,
                "debug_group_layer_indices": [int(i) for i in layer_indices],
                "debug_recent_count": _recent(int(items[n]["total_tokens"])),
                "cache_len_after": k,
            }
        return out

    setattr(_select_keep_indices, "_supports_paged", True)
    setattr(_select_keep_indices_for_group_per_head, "_supports_paged_group", True)
    setattr(_select_keep_indices_for_group_per_head, "_fused_group_compress", _compress_group_fused)
    setattr(_select_keep_indices_for_group_per_head, "_fused_group_compress_batch", _compress_group_fused_batch)
    return _select_keep_indices, _select_keep_indices_for_group_per_head, "enabled"
