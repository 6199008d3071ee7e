"""Runs the reference's OWN CPU code for the path (score -> select -> compact) from ``oracle/_ref``.

TEST / BASELINE INFRASTRUCTURE ONLY: used by ``bench.py`` (the ``cpu_baseline`` leg and ``--impl reference``)
and by tests, never by the product package.  ``oracle/_ref`` holds an unmodified copy of the reference's
Python packages made by ``oracle/build_ref.py``.  The code is imported as is, with the three shims the
fixture generator also uses, because the selector insists on a GPU:

1. ``compute_scores_triton`` (called unconditionally, runtime/selector_hf.py:59,314) is pointed at the
   reference's own ``compute_scores_pytorch`` on ``K.float()`` (the Triton kernel upcasts K in-kernel,
   core/kernels/triton_scoring.py:263-264);
2. ``TriAttentionConfig`` defaults to ``device='cpu'`` (core/config.py:85 says cuda);
3. the statistics file carries ``inv_freq`` so that no model config is fetched from the Hub.
"""
from __future__ import annotations

import sys
import tempfile
import time
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"
_state: dict = {}


def available() -> bool:
    return (REF_DIR / "triattention" / "vllm" / "runtime" / "selector_hf.py").is_file()


def _load(gpu: bool = False):
    """Import the reference from oracle/_ref.  ``gpu=False`` installs the CPU shims; ``gpu=True`` leaves the
    reference untouched (its Triton scorer, CUDA tensors) - one process uses one of the two."""
    if _state:
        if _state["gpu"] != gpu:
            raise RuntimeError("the reference was already imported for the other device in this process")
        return _state
    if not available():
        raise RuntimeError("oracle/_ref is absent: run `python oracle/build_ref.py` where a reference checkout is mounted")
    sys.dont_write_bytecode = True
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import triattention.vllm.core.config as ref_config
    import triattention.vllm.core.scoring as ref_scoring

    if gpu:
        import triattention.vllm.runtime.config as ref_runtime_config
        from triattention.vllm.runtime.kv_compaction import compact_request_kv_in_place_per_head
        from triattention.vllm.runtime.selector_hf import build_triattention_selector
        _state.update(gpu=True, runtime_config=ref_runtime_config, build_selector=build_triattention_selector,
                      compact_per_head=compact_request_kv_in_place_per_head)
        return _state
    pyt = ref_scoring.compute_scores_pytorch

    def _triton_shim(**kw):
        kw.pop("trig_cache", None)
        kw["key_states"] = kw["key_states"].float()
        return pyt(**kw)

    ref_scoring.compute_scores_triton = _triton_shim
    if not getattr(ref_config.TriAttentionConfig, "_cpu_default_installed", False):
        orig_init = ref_config.TriAttentionConfig.__init__

        def _init(self, *a, **kw):
            kw.setdefault("device", torch.device("cpu"))
            orig_init(self, *a, **kw)

        ref_config.TriAttentionConfig.__init__ = _init
        ref_config.TriAttentionConfig._cpu_default_installed = True
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.kv_compaction import compact_request_kv_in_place_per_head
    from triattention.vllm.runtime.selector_hf import build_triattention_selector

    _state.update(gpu=False, runtime_config=ref_runtime_config, build_selector=build_triattention_selector,
                  compact_per_head=compact_request_kv_in_place_per_head)
    return _state


def make_group_selector(stats_path, budget: int, window: int, aggregation: str = "mean", gpu: bool = False):
    """The reference's group selector (runtime/selector_hf.py:749-1083) for a statistics file on disk."""
    st = _load(gpu)
    cfg = st["runtime_config"].TriAttentionRuntimeConfig(
        kv_budget=int(budget), window_size=int(window), sparse_stats_path=Path(stats_path),
        sparse_score_aggregation=aggregation)
    cfg.validate()
    _, sel_group, status = st["build_selector"](cfg)
    if status != "enabled":
        raise RuntimeError(f"reference selector not enabled: {status}")
    return sel_group


def select_and_compact(sel_group, caches, block_ids, block_size: int, total_tokens: int, round_start: int, budget: int):
    """One request through the reference: group selection over ``caches`` (one 5-D paged tensor per layer, CPU)
    and its per-layer in-place compaction (runtime/kv_compaction.py:461-599, dropped tokens preserved as
    runtime/layout_engine.py:71-80 forces).  Returns (keep [Hkv, k] int64, seconds)."""
    st = _state if _state else _load()

    def _iter():
        for l, c in enumerate(caches):
            yield l, c, block_ids, block_size

    on_gpu = bool(caches) and caches[0].is_cuda
    if on_gpu:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, total_tokens=int(total_tokens),
                    prefill_len=0, protect_prefill=False, round_start=int(round_start),
                    budget_total=min(int(budget), int(total_tokens)))
    keep = res["indices"]
    bt = torch.as_tensor(block_ids, dtype=torch.long, device=caches[0].device)
    for c in caches:
        st["compact_per_head"](kv_cache=c, block_ids=bt, block_size=block_size, keep_token_indices_per_head=keep,
                               total_tokens=int(total_tokens), preserve_dropped_tokens=True)
    if on_gpu:
        torch.cuda.synchronize()
    return keep, time.perf_counter() - t0


def stats_file(tmp_dir, save_fn, stats) -> Path:
    """Write ``stats`` (with inv_freq in the metadata) where the reference's loader can read it."""
    p = Path(tmp_dir) / "stats.pt"
    save_fn(stats, p)
    return p
