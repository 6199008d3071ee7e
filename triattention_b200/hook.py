"""Runner compression hook with the contract of the reference's runtime/hook_impl.py.

``install_runner_compression_hook(base_runner, config)`` sets ``base_runner.triattention_apply_compression``;
the hook is called as ``hook(req_id=..., signal=..., scheduler_output=...)`` and returns the same result dict
(keys and reason strings of hook_impl.py:96-112, hook_preflight.py:203-234, hook_group_pipeline.py:100-148,
plan_models.py:121-134).  Selection and compaction run on the CUDA kernels: in the default mode
(per-KV-head keep set shared by all layers) one fused native call handles a whole KV-cache group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from .config import TriAttentionRuntimeConfig
from .constants import TRITON_SCORING_REQUIRED_MARKER
from .kv_compaction import (build_keep_token_indices, compact_group_kv_in_place_per_head,
                            compact_request_kv_in_place, compact_request_kv_in_place_per_head,
                            register_kv_layout_axis_hint)
from .layout_engine import num_required_blocks, truncate_tail_reclaim_group
from .perf_profile import HookPerfProfile
from .plan_models import KeepPlan, PlacementPlan, ReclaimEvent
from .request_state import resolve_hook_request_context, scheduled_tokens_for_req
from .selector import FusedCompactionError, build_triattention_selector as _build_triattention_selector
from .signals import CompressionSignal


# the native per-layer compaction; a caller that injects another function keeps the per-layer loop
_NATIVE_PER_HEAD_COMPACT = compact_request_kv_in_place_per_head


# ------------------------------------------------------------------------------------------ runtime context
@dataclass(frozen=True)
class HookRuntimeContext:
    scheduled_tokens: int
    num_computed_tokens: int
    estimated_effective_tokens: int
    effective_tokens: int
    budget_total: int
    recent_unabsorbed_tokens: Optional[int]
    should_defer_recompress: bool


def effective_budget_for_signal(config, signal, total_tokens: int) -> int:
    """min(T, kv_budget [+ prefill when it is protected outside the budget]) (hook_runtime_context.py:14-22)."""
    budget = config.kv_budget
    if signal.protect_prefill and not config.include_prefill_in_budget:
        budget += max(signal.prefill_len, 0)
    return min(total_tokens, budget)


def build_hook_runtime_context(*, base_runner, config, req_id, req_state, req_runtime_state, signal,
                               scheduler_output, compressed_once: set, original_block_ids_by_group,
                               block_size_hint: int) -> HookRuntimeContext:
    """Effective cached length, budget and the re-compression gate (hook_runtime_context.py:106-209)."""
    capacity = None
    if block_size_hint > 0 and isinstance(original_block_ids_by_group, (list, tuple)):
        caps = [len(g) * block_size_hint for g in original_block_ids_by_group if isinstance(g, (list, tuple))]
        capacity = min(caps) if caps else None
    scheduled = scheduled_tokens_for_req(scheduler_output, req_id)
    num_computed = int(getattr(req_state, "num_computed_tokens", 0))
    estimated = max(0, int(getattr(signal, "estimated_cache_len", 0)))
    if req_runtime_state is not None:
        count = getattr(req_runtime_state, "compression_count", None)
        cur = getattr(req_runtime_state, "current_cache_len", None)
        if isinstance(count, int) and count > 0 and isinstance(cur, int) and cur > 0:
            estimated = max(0, int(cur))
    post_forward = getattr(signal, "_post_forward", False)
    effective = max(0, estimated) if post_forward else max(0, estimated - max(0, scheduled))
    effective = min(effective, num_computed + (scheduled if post_forward else 0))
    if isinstance(capacity, int):
        effective = min(effective, capacity + block_size_hint)
    recent = None
    if req_runtime_state is not None:
        recent = max(0, effective - int(getattr(req_runtime_state, "last_absorbed_cache_len", 0)))
    setattr(base_runner, "_triattention_active_recent_unabsorbed_tokens", recent)

    prefill_len = int(getattr(signal, "prefill_len", 0) or 0)
    prefill_incomplete = prefill_len > 0 and num_computed < prefill_len
    if (config.fail_on_effective_len_regression and config.enable_experimental_block_reclaim
            and req_id in compressed_once and not prefill_incomplete):
        budget = config.kv_budget
        if signal.protect_prefill and not config.include_prefill_in_budget:
            budget += max(signal.prefill_len, 0)
        guard_upper = budget + max(1, config.effective_len_guard_divide_multiples) * max(1, config.divide_length)
        est_slack = max(1, int(getattr(signal, "estimated_cache_len", 0)) - num_computed)
        slack = block_size_hint + est_slack + max(1, scheduled)
        if (effective > guard_upper + slack and num_computed > guard_upper + slack
                and effective >= int(config.effective_len_regression_ratio * num_computed)):
            raise RuntimeError(
                f"{TRITON_SCORING_REQUIRED_MARKER}:effective_len_regressed:req={req_id}:"
                f"effective_tokens={effective}:num_computed_tokens={num_computed}:guard_upper={guard_upper}")

    budget_total = effective_budget_for_signal(config, signal, effective)
    gate_hit = estimated >= budget_total + max(1, config.divide_length)
    kv_override = str(getattr(signal, "reason", "")) == "kv_usage_threshold"
    defer = bool(config.enable_experimental_kv_compaction and req_id in compressed_once
                 and not kv_override and not gate_hit)
    return HookRuntimeContext(int(scheduled), int(num_computed), int(estimated), int(effective), int(budget_total),
                              int(recent) if isinstance(recent, int) else None, defer)


# ------------------------------------------------------------------------------------------ group tensors
def _infer_layer_idx(name: str, layer: Any, fallback: int) -> int:
    import re
    for attr in ("layer_idx", "layer_id", "idx"):
        v = getattr(layer, attr, None)
        if isinstance(v, int):
            return v
    m = re.findall(r"\d+", name)
    return int(m[-1]) if m else fallback


def _infer_kv_axis(base_runner: Any, gid: int) -> Optional[int]:
    """K/V axis of a group's cache tensors from its attention backend (kv_group_resolver.py:24-65)."""
    groups = getattr(base_runner, "attn_groups", None)
    if not isinstance(groups, (list, tuple)) or not (0 <= gid < len(groups)):
        return None
    backend = getattr(groups[gid], "backend", None)
    if backend is None:
        return None
    cls = backend if isinstance(backend, type) else backend.__class__
    shape_fn = getattr(cls, "get_kv_cache_shape", None)
    if callable(shape_fn):
        try:
            shape = tuple(int(x) for x in shape_fn(3, 16, 1, 1))  # 3 blocks: no (2, 2, ...) ambiguity
            if len(shape) >= 2 and ((shape[0] == 2) ^ (shape[1] == 2)):
                return 0 if shape[0] == 2 else 1
        except Exception:
            pass
    ident = f"{getattr(cls, '__module__', '')}.{getattr(cls, '__name__', '')}".lower()
    if "flash_attn" in ident:
        return 0
    if "triton_attn" in ident:
        return 1
    return None


def resolve_group_tensors(base_runner: Any) -> dict:
    """gid -> [(layer_idx, kv_cache)] from the runner (kv_group_resolver.py:68-141)."""
    out: dict = {}
    kv_cache_config = getattr(base_runner, "kv_cache_config", None)
    comp = getattr(base_runner, "compilation_config", None)
    ctx = getattr(comp, "static_forward_context", None) if comp is not None else None
    if kv_cache_config is None or not isinstance(ctx, dict):
        fallback = getattr(base_runner, "kv_caches", None)
        if isinstance(fallback, list):
            tensors = [(i, t) for i, t in enumerate(fallback) if isinstance(t, torch.Tensor)]
            if tensors:
                out[0] = tensors
        return out
    groups = getattr(kv_cache_config, "kv_cache_groups", None)
    if not isinstance(groups, (list, tuple)):
        return out
    for gid, group in enumerate(groups):
        names = getattr(group, "layer_names", None)
        if not isinstance(names, (list, tuple)):
            continue
        tensors, seen = [], set()
        for local, name in enumerate(names):
            layer = ctx.get(name)
            caches = getattr(layer, "kv_cache", None) if layer is not None else None
            if not isinstance(caches, list) or not caches or not isinstance(caches[0], torch.Tensor):
                continue
            t = caches[0]
            if t.data_ptr() in seen:
                continue
            seen.add(t.data_ptr())
            tensors.append((_infer_layer_idx(name, layer, local), t))
        if tensors:
            axis = _infer_kv_axis(base_runner, gid)
            if axis is not None:
                for _, t in tensors:
                    try:
                        register_kv_layout_axis_hint(t, axis)
                    except ValueError:
                        pass
            out[gid] = tensors
    return out


# ------------------------------------------------------------------------------------------ group pipeline
@dataclass
class _Pending:
    """A request that passed the host-side checks of the hook and is about to be compacted."""
    req_id: Any
    signal: Any
    strict: bool
    rt: Any
    req_state: Any
    original_ids: Any
    mutable: list
    block_size: int


@dataclass(frozen=True)
class GroupPipelineOutcome:
    cache_len_after: int
    selection_mode: str
    block_reclaim_groups: list
    mutable_block_ids_by_group: list


def _select_for_group(*, req_id, gid, layer_tensors, block_ids, block_size, total_tokens, prefill_len,
                      protect_prefill, round_start, budget_total, config, strict, select_keep_indices,
                      select_keep_indices_for_group):
    """[(layer_idx, kv_cache, KeepPlan)] and the selection-mode label (selection_planner.py:94-275)."""
    group_result = None
    if (select_keep_indices_for_group is not None and config.pruning_mode == "per_head"
            and config.per_head_selection_semantics == "hf_aligned_global_per_head"):
        try:
            if strict and not getattr(select_keep_indices_for_group, "_supports_paged_group", False):
                raise RuntimeError("paged_group_selector_required")

            def _iter_kv():
                for layer_idx, kv_cache in layer_tensors:
                    yield layer_idx, kv_cache, block_ids, block_size

            group_result = select_keep_indices_for_group(
                layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter_kv, total_tokens=total_tokens,
                prefill_len=prefill_len, protect_prefill=protect_prefill, round_start=round_start,
                budget_total=budget_total)
        except Exception as exc:
            raise RuntimeError(
                f"{TRITON_SCORING_REQUIRED_MARKER}:req={req_id}:gid={gid}:global_per_head:{type(exc).__name__}") from exc
    tasks, label = [], "fallback"
    for layer_idx, kv_cache in layer_tensors:
        selected = group_result
        if selected is None and select_keep_indices is not None:
            try:
                if strict and not getattr(select_keep_indices, "_supports_paged", False):
                    raise RuntimeError("paged_selector_required")
                selected = select_keep_indices(
                    keys_dense=None, kv_cache=kv_cache, block_ids=block_ids, block_size=block_size,
                    total_tokens=total_tokens, prefill_len=prefill_len, protect_prefill=protect_prefill,
                    layer_idx=layer_idx, round_start=round_start, budget_total=budget_total)
            except Exception as exc:
                raise RuntimeError(
                    f"{TRITON_SCORING_REQUIRED_MARKER}:req={req_id}:gid={gid}:layer={layer_idx}:{type(exc).__name__}") from exc
        from_fallback = False
        if selected is None:
            keep = build_keep_token_indices(total_tokens, config.kv_budget, prefill_len, protect_prefill,
                                            config.include_prefill_in_budget)
            if keep is None:
                raise ValueError("prefill_exceeds_budget")
            if strict:
                raise RuntimeError(
                    f"{TRITON_SCORING_REQUIRED_MARKER}:selector_returned_none:req={req_id}:gid={gid}:layer={layer_idx}")
            selected = {"mode": "shared", "indices": keep}
            from_fallback = True
        plan = KeepPlan.from_selector_result(selected)
        label = "fallback" if from_fallback else plan.selection_mode_label
        tasks.append((layer_idx, kv_cache, plan))
    return tasks, label


def run_group_compaction_pipeline(*, req_id, signal, config, strict, num_computed_tokens, effective_tokens,
                                  budget_total, block_size, mutable_block_ids_by_group, group_tensors,
                                  select_keep_indices, select_keep_indices_for_group, shared_compact_fn,
                                  per_head_compact_fn, fused_results: Optional[dict] = None):
    """Select and compact every KV-cache group of one request (hook_group_pipeline.py:42-155).

    ``fused_results`` maps a group id to the result of a fused native step that has ALREADY run for this request
    (the batched hook runs it for several requests at once); such a group is only finished here."""
    compacted_any = False
    cache_len_after = None
    label = "fallback"
    reclaim_groups = []
    for gid, block_ids in enumerate(mutable_block_ids_by_group):
        if not block_ids:
            continue
        layer_tensors = group_tensors.get(gid)
        if not layer_tensors:
            continue
        total = min(effective_tokens, len(block_ids) * block_size)
        if total <= 0:
            continue
        prefill_len = min(int(signal.prefill_len), total)
        group_budget = min(budget_total, total)
        round_start = int(max(0, num_computed_tokens))
        # Default mode with the native selector and the native compaction: one fused call does the whole group.
        fused = getattr(select_keep_indices_for_group, "_fused_group_compress", None)
        fused_result = None
        if fused_results is not None and gid in fused_results:
            fused_result = fused_results[gid]
        elif (fused is not None and per_head_compact_fn is _NATIVE_PER_HEAD_COMPACT
                and not bool(getattr(config, "preserve_dropped_tokens", False))
                and config.pruning_mode == "per_head"
                and config.per_head_selection_semantics == "hf_aligned_global_per_head"
                and len({t.device for _, t in layer_tensors}) == 1):
            try:
                fused_result = fused(
                    caches=[t for _, t in layer_tensors], layer_indices=[i for i, _ in layer_tensors],
                    block_ids=block_ids, total_tokens=total, prefill_len=prefill_len,
                    protect_prefill=signal.protect_prefill, round_start=round_start, budget_total=group_budget)
            except FusedCompactionError as exc:
                first = layer_tensors[0][0] if layer_tensors else -1
                return {"applied": False, "reason": f"compaction_failed:g{gid}:l{first}:{type(exc).__name__}"}
            except Exception as exc:
                raise RuntimeError(
                    f"{TRITON_SCORING_REQUIRED_MARKER}:req={req_id}:gid={gid}:global_per_head:{type(exc).__name__}") from exc
        try:
            if fused_result is not None:
                tasks, label = [], KeepPlan.from_selector_result(fused_result).selection_mode_label
            else:
                tasks, label = _select_for_group(
                    req_id=req_id, gid=gid, layer_tensors=layer_tensors, block_ids=block_ids, block_size=block_size,
                    total_tokens=total, prefill_len=prefill_len, protect_prefill=signal.protect_prefill,
                    round_start=round_start, budget_total=group_budget, config=config, strict=strict,
                    select_keep_indices=select_keep_indices, select_keep_indices_for_group=select_keep_indices_for_group)
        except ValueError as exc:
            if str(exc) == "prefill_exceeds_budget":
                return {"applied": False, "reason": "prefill_exceeds_budget"}
            raise
        group_len = int(fused_result["cache_len_after"]) if fused_result is not None else None
        layer_lens: list = []
        try:
            bt_cache: dict = {}
            preserve = bool(getattr(config, "preserve_dropped_tokens", False))
            one_plan = (fused_result is None and len(tasks) > 1 and tasks[0][2].mode == "per_head"
                        and all(t[2] is tasks[0][2] or t[2].indices is tasks[0][2].indices for t in tasks)
                        and per_head_compact_fn is _NATIVE_PER_HEAD_COMPACT
                        and len({t[1].device for t in tasks}) == 1)
            if one_plan:
                # one keep set for every layer of the group: a single launch compacts all layers
                group_len = int(compact_group_kv_in_place_per_head(
                    [t[1] for t in tasks], block_ids, block_size, tasks[0][2].indices, total, preserve))
                tasks_to_run = []
            else:
                tasks_to_run = tasks
            for layer_idx, kv_cache, plan in tasks_to_run:
                bt = bt_cache.get(kv_cache.device)
                if bt is None:
                    bt = torch.as_tensor(block_ids, device=kv_cache.device, dtype=torch.long)
                    bt_cache[kv_cache.device] = bt
                if plan.mode == "per_head":
                    n = per_head_compact_fn(kv_cache=kv_cache, block_ids=bt, block_size=block_size,
                                            keep_token_indices_per_head=plan.indices, total_tokens=total,
                                            preserve_dropped_tokens=preserve)
                else:
                    n = shared_compact_fn(kv_cache=kv_cache, block_ids=bt, block_size=block_size,
                                          keep_token_indices=plan.indices, total_tokens=total,
                                          preserve_dropped_tokens=preserve)
                layer_lens.append((layer_idx, int(n)))
                if group_len is None:
                    group_len = int(n)
            kept_ids, removed_ids, reclaim = list(block_ids), [], None
            if config.enable_experimental_block_reclaim and group_len is not None:
                kept_ids, removed_ids, reclaim = truncate_tail_reclaim_group(
                    gid=gid, normalized_block_ids=block_ids, cache_len_after=group_len, block_size=block_size)
                if config.require_physical_reclaim:
                    expect = max(0, num_required_blocks(total, block_size) - num_required_blocks(group_len, block_size))
                    if expect > 0 and len(removed_ids) < expect:
                        raise RuntimeError(
                            f"{TRITON_SCORING_REQUIRED_MARKER}:physical_reclaim_missing:req={req_id}:gid={gid}:"
                            f"expected_removed>={expect}:actual_removed={len(removed_ids)}:"
                            f"effective_tokens={total}:cache_len_after={group_len}")
        except Exception as exc:
            first = tasks[0][0] if tasks else -1
            return {"applied": False, "reason": f"compaction_failed:g{gid}:l{first}:{type(exc).__name__}"}
        # every layer of every group must end at the same length; a mismatch is fatal, not a soft
        # compaction failure (hook_group_pipeline.py:128-135 raises it outside the try block)
        for layer_idx, n in layer_lens:
            expect = cache_len_after if cache_len_after is not None else group_len
            if n != expect:
                raise RuntimeError(
                    f"{TRITON_SCORING_REQUIRED_MARKER}:inconsistent_cache_len_after:req={req_id}:gid={gid}:"
                    f"layer={layer_idx}:expected={expect}:actual={n}")
        if group_len is not None:
            if cache_len_after is not None and group_len != cache_len_after:
                raise RuntimeError(
                    f"{TRITON_SCORING_REQUIRED_MARKER}:inconsistent_cache_len_after:req={req_id}:gid={gid}:"
                    f"layer={tasks[0][0] if tasks else -1}:expected={cache_len_after}:actual={group_len}")
            cache_len_after = group_len
            compacted_any = True
            if config.enable_experimental_block_reclaim:
                mutable_block_ids_by_group[gid] = kept_ids
                if reclaim is not None:
                    reclaim_groups.append(reclaim)
    if not compacted_any or cache_len_after is None:
        return {"applied": False, "reason": "no_compactable_groups"}
    return GroupPipelineOutcome(int(cache_len_after), str(label), reclaim_groups, mutable_block_ids_by_group)


def fused_step_allowed(config, per_head_compact_fn=_NATIVE_PER_HEAD_COMPACT) -> bool:
    """Configuration under which a KV-cache group is handled by the fused native step (default mode)."""
    return (per_head_compact_fn is _NATIVE_PER_HEAD_COMPACT
            and not bool(getattr(config, "preserve_dropped_tokens", False))
            and config.pruning_mode == "per_head"
            and config.per_head_selection_semantics == "hf_aligned_global_per_head")


def compactable_groups(*, signal, num_computed_tokens, effective_tokens, budget_total, block_size,
                       mutable_block_ids_by_group, group_tensors) -> list:
    """The groups run_group_compaction_pipeline would work on, with the arguments of their selection step:
    ``[(gid, layer_tensors, item)]``, item = keyword arguments of the fused step other than the tensors."""
    out = []
    for gid, block_ids in enumerate(mutable_block_ids_by_group):
        if not block_ids:
            continue
        layer_tensors = group_tensors.get(gid)
        if not layer_tensors:
            continue
        total = min(effective_tokens, len(block_ids) * block_size)
        if total <= 0:
            continue
        out.append((gid, layer_tensors, dict(
            block_ids=block_ids, total_tokens=total, prefill_len=min(int(signal.prefill_len), total),
            protect_prefill=signal.protect_prefill, round_start=int(max(0, num_computed_tokens)),
            budget_total=min(budget_total, total))))
    return out


# ------------------------------------------------------------------------------------------ hook factory
def make_runner_compression_hook(base_runner: Any, config: TriAttentionRuntimeConfig) -> Callable[..., dict]:
    """Create the hook bound to ``base_runner`` (hook_impl.py:29-165)."""
    try:
        sel_layer, sel_group, selector_status = _build_triattention_selector(config, base_runner=base_runner)
    except TypeError:
        sel_layer, sel_group, selector_status = _build_triattention_selector(config)
    cache: dict = {"group_tensors": None}
    compressed_once: set = set()

    def _plan(req_id: str, signal: CompressionSignal, scheduler_output: Any):
        """Host-side part of a call up to the point where the cache is touched: a result dictionary when the
        request is skipped, otherwise what the compaction step needs."""
        setattr(base_runner, "_triattention_active_req_id", req_id)
        strict = bool(config.enable_experimental_kv_compaction and config.require_triton_scoring)
        ctx = resolve_hook_request_context(base_runner=base_runner, req_id=req_id, scheduler_output=scheduler_output)
        if isinstance(ctx, dict):
            return ctx
        req_state = ctx.req_state
        block_size_hint = int(getattr(getattr(base_runner, "cache_config", None), "block_size", 0))
        if block_size_hint <= 0:
            block_size_hint = 1
        original_ids = getattr(req_state, "block_ids", None)
        rt = build_hook_runtime_context(
            base_runner=base_runner, config=config, req_id=req_id, req_state=req_state,
            req_runtime_state=ctx.req_runtime_state, signal=signal, scheduler_output=scheduler_output,
            compressed_once=compressed_once, original_block_ids_by_group=original_ids,
            block_size_hint=block_size_hint)
        if rt.effective_tokens <= rt.budget_total or rt.should_defer_recompress:
            return {"applied": False, "reason": "under_budget", "cache_len_after": rt.effective_tokens}
        if not config.enable_experimental_kv_compaction:
            plan = build_keep_token_indices(rt.effective_tokens, config.kv_budget, signal.prefill_len,
                                            signal.protect_prefill, config.include_prefill_in_budget)
            if plan is None:
                return {"applied": False, "reason": "prefill_exceeds_budget"}
            return {"applied": False, "reason": "plan_only", "cache_len_after": len(plan)}
        if strict and sel_layer is None:
            raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:selector_unavailable:{selector_status}")

        kv_caches = getattr(base_runner, "kv_caches", None)
        cache_config = getattr(base_runner, "cache_config", None)
        if not isinstance(kv_caches, list) or cache_config is None:
            return {"applied": False, "reason": "kv_cache_unavailable"}
        block_size = int(getattr(cache_config, "block_size", 0))
        if block_size <= 0:
            return {"applied": False, "reason": "invalid_block_size"}
        if not original_ids:
            return {"applied": False, "reason": "missing_block_ids"}
        if not isinstance(original_ids, (list, tuple)):
            return {"applied": False, "reason": "invalid_block_ids_container"}
        mutable = [[int(b) for b in g] if isinstance(g, (list, tuple)) else None for g in original_ids]
        if cache["group_tensors"] is None:
            cache["group_tensors"] = resolve_group_tensors(base_runner)
        return _Pending(req_id=req_id, signal=signal, strict=strict, rt=rt, req_state=req_state,
                        original_ids=original_ids, mutable=mutable, block_size=block_size)

    def _finish(p: "_Pending", fused_results: Optional[dict] = None) -> dict:
        """Selection, compaction and bookkeeping of one planned request."""
        rt, original_ids, req_state = p.rt, p.original_ids, p.req_state
        setattr(base_runner, "_triattention_active_req_id", p.req_id)
        out = run_group_compaction_pipeline(
            req_id=p.req_id, signal=p.signal, config=config, strict=p.strict, num_computed_tokens=rt.num_computed_tokens,
            effective_tokens=rt.effective_tokens, budget_total=rt.budget_total, block_size=p.block_size,
            mutable_block_ids_by_group=p.mutable, group_tensors=cache["group_tensors"],
            select_keep_indices=sel_layer, select_keep_indices_for_group=sel_group,
            shared_compact_fn=compact_request_kv_in_place, per_head_compact_fn=compact_request_kv_in_place_per_head,
            fused_results=fused_results)
        if isinstance(out, dict):
            return out
        compressed_once.add(p.req_id)

        reclaim_event = None
        if config.enable_experimental_block_reclaim and out.block_reclaim_groups:
            new_ids = [original_ids[i] if g is None else g for i, g in enumerate(out.mutable_block_ids_by_group)]
            req_state.block_ids = tuple(new_ids) if isinstance(original_ids, tuple) else new_ids
            reclaim_event = ReclaimEvent(mode="truncate_tail", groups=out.block_reclaim_groups)
        return PlacementPlan(
            cache_len_after=out.cache_len_after, selector_status=str(selector_status),
            selection_mode=out.selection_mode, effective_tokens_before=rt.effective_tokens,
            budget_total=rt.budget_total, recent_unabsorbed_tokens=rt.recent_unabsorbed_tokens,
            block_reclaim=reclaim_event).to_hook_result_dict()

    def _hook(req_id: str, signal: CompressionSignal, scheduler_output: Any) -> dict:
        p = _plan(req_id, signal, scheduler_output)
        return p if isinstance(p, dict) else _finish(p)

    def _hook_batch(requests, scheduler_output: Any) -> dict:
        """All triggered requests of a step: ``requests`` = [(req_id, signal), ...]; returns {req_id: result} with
        the dictionaries the per-request hook would return, in one native call for every request that is in the
        default mode and has a single compactable KV-cache group (the others go through the per-request path)."""
        results: dict = {}
        pending = []
        for req_id, signal in requests:
            p = _plan(req_id, signal, scheduler_output)
            if isinstance(p, dict):
                results[req_id] = p
            else:
                pending.append(p)
        fused_batch = getattr(sel_group, "_fused_group_compress_batch", None)
        fused_for: dict = {}   # req_id -> {gid: selector result}
        failed: dict = {}      # req_id -> soft failure result
        if fused_batch is not None and fused_step_allowed(config) and len(pending) > 1:
            by_group: dict = {}
            for p in pending:
                groups = compactable_groups(
                    signal=p.signal, num_computed_tokens=p.rt.num_computed_tokens, effective_tokens=p.rt.effective_tokens,
                    budget_total=p.rt.budget_total, block_size=p.block_size, mutable_block_ids_by_group=p.mutable,
                    group_tensors=cache["group_tensors"])
                if len(groups) == 1 and len({t.device for _, t in groups[0][1]}) == 1:
                    gid, layer_tensors, item = groups[0]
                    by_group.setdefault(gid, (layer_tensors, []))[1].append((p, item))
            for gid, (layer_tensors, members) in by_group.items():
                if len(members) < 2:
                    continue
                try:
                    outs = fused_batch(caches=[t for _, t in layer_tensors], layer_indices=[i for i, _ in layer_tensors],
                                       items=[item for _, item in members])
                except FusedCompactionError as exc:
                    first = layer_tensors[0][0] if layer_tensors else -1
                    for p, _ in members:
                        failed[p.req_id] = {"applied": False,
                                            "reason": f"compaction_failed:g{gid}:l{first}:{type(exc).__name__}"}
                    continue
                except Exception as exc:
                    raise RuntimeError(f"{TRITON_SCORING_REQUIRED_MARKER}:req={members[0][0].req_id}:gid={gid}:"
                                       f"global_per_head:{type(exc).__name__}") from exc
                for (p, _), res in zip(members, outs):
                    if res is not None:
                        fused_for[p.req_id] = {gid: res}
        for p in pending:
            results[p.req_id] = failed.get(p.req_id) or _finish(p, fused_for.get(p.req_id))
        return results

    # TRIATTN_RUNTIME_PERF_PROFILE / TRIATTN_RUNTIME_NVTX: aggregated TRIATTN_PERF lines, NVTX range per call
    wrapped = HookPerfProfile.from_env().wrap(_hook)
    setattr(wrapped, "batch", _hook_batch)
    return wrapped


def install_runner_compression_hook(base_runner: Any, config: TriAttentionRuntimeConfig) -> None:
    """Install the hook on the runner unless one is already present (hook_impl.py:174-185)."""
    if hasattr(base_runner, "triattention_apply_compression"):
        return
    hook = make_runner_compression_hook(base_runner=base_runner, config=config)
    setattr(base_runner, "triattention_apply_compression", hook)
    # all triggered requests of a step in one call (no counterpart in the reference, whose worker loops over them)
    setattr(base_runner, "triattention_apply_compression_batch", getattr(hook, "batch", None))
