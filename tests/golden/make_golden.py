#!/usr/bin/env python
"""Generate the golden fixtures in this directory from the reference itself.

Run where a checkout of the reference is available (default: a directory
``reference`` next to this repository, override with ``TRIATTN_REFERENCE_ROOT``)::

    python tests/golden/make_golden.py                       # everything
    python tests/golden/make_golden.py --only input_patch    # only input_patch_cases.npz
    python tests/golden/make_golden.py --only calibration    # only calibration_cases.npz
    python tests/golden/make_golden.py --only bench_shapes   # only bench_shape_cases.npz (minutes of CPU time)
    python tests/golden/make_golden.py --only shipped_stats  # only shipped_stats_cases.npz
    python tests/golden/make_golden.py --only stats_loader   # only the stats_loader_cases entry of manifest.json
    python tests/golden/make_golden.py --only runner_actions # only runner_action_cases.json
    python tests/golden/make_golden.py --only state_store    # only state_store_cases.json
    python tests/golden/make_golden.py --only effective_overrides  # only effective_override_cases.json
    python tests/golden/make_golden.py --only step_lifecycle # only step_lifecycle_cases.json
    python tests/golden/make_golden.py --only scheduler_side # only scheduler_side_cases.json
    python tests/golden/make_golden.py --only worker_runner  # only worker_runner_cases.json
    python tests/golden/make_golden.py --only input_patch_closures  # only input_patch_closure_cases.json

The reference is imported unmodified, on CPU, with three test-side shims:

1. ``triattention.vllm.core.scoring.compute_scores_triton`` is replaced by the
   reference's own ``compute_scores_pytorch`` applied to ``K.float()`` (the
   selector calls the Triton entry unconditionally, selector_hf.py:59,314; the
   Triton kernel upcasts K in-kernel, triton_scoring.py:263-264).
2. ``TriAttentionConfig`` defaults to ``device='cpu'`` (core/config.py:85 says cuda).
3. ``inv_freq`` is stored in the stats metadata so no model config is fetched.

Each fixture stores the seeds/parameters that regenerate the inputs with
``triattention_b200.synth`` plus a SHA-256 of those inputs, and the
reference's outputs.  Tiny cases also store the inputs themselves.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(os.environ.get("TRIATTN_REFERENCE_ROOT", str(REPO.parent / "reference")))
sys.dont_write_bytecode = True
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "tests"))
sys.path.insert(0, str(REF))

import synth  # noqa: E402


def sha(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def bf16_to_np(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def install_shims():
    import triattention.vllm.core.scoring as ref_scoring
    import triattention.vllm.core.config as ref_config

    pyt = ref_scoring.compute_scores_pytorch

    def _triton_shim(**kw):
        kw.pop("trig_cache", None)
        kw["key_states"] = kw["key_states"].float()
        return pyt(**kw)

    ref_scoring.compute_scores_triton = _triton_shim
    orig_init = ref_config.TriAttentionConfig.__init__

    def _init(self, *a, **kw):
        kw.setdefault("device", torch.device("cpu"))
        orig_init(self, *a, **kw)

    ref_config.TriAttentionConfig.__init__ = _init
    return ref_scoring, ref_config


# --------------------------------------------------------------------------
# Case builders (shared with the tests through the stored parameters)
# --------------------------------------------------------------------------

def build_paged_case(p: dict):
    """Regenerate (stats, layer caches, block ids) from the parameter dict ``p``."""
    gen = torch.Generator().manual_seed(int(p["seed"]))
    inv_freq = synth.rope_inv_freq(p["head_dim"], p["theta"], p.get("llama3"))
    stats = synth.make_stats(p["num_layers"], p["num_q_heads"], p["head_dim"], inv_freq, gen,
                             rope_style=p.get("rope_style", "half"))
    T = p["total_tokens"]
    bs = p["block_size"]
    nblk = (T + bs - 1) // bs
    nb_total = nblk + p.get("spare_blocks", 5)
    if p.get("consecutive_blocks", False):
        block_ids = list(range(2, 2 + nblk))
        nb_total = max(nb_total, 2 + nblk)
    else:
        block_ids = synth.random_block_ids(nblk, nb_total, gen)
    caches = []
    for _l in range(p["num_layers"]):
        cache = synth.make_paged_layer(nb_total, bs, p["num_kv_heads"], p["head_dim"], kv_axis=p["kv_axis"])
        k = synth.make_rotated_keys(p["num_kv_heads"], T, p["head_dim"], inv_freq, gen,
                                    rope_style=p.get("rope_style", "half"))
        v = synth.make_values(p["num_kv_heads"], T, p["head_dim"], gen)
        synth.write_tokens_to_paged(cache, p["kv_axis"], block_ids, bs, k, v)
        caches.append(cache)
    return stats, caches, block_ids


def runtime_config(ref_runtime_config, stats_path, p):
    cfg = ref_runtime_config.TriAttentionRuntimeConfig(
        kv_budget=p["budget"],
        window_size=p["window"],
        sparse_stats_path=Path(stats_path),
        sparse_score_aggregation=p.get("aggregation", "mean"),
        sparse_normalize_scores=p.get("normalize", True),
        pruning_mode=p.get("pruning_mode", "per_head"),
        per_head_selection_semantics=p.get("semantics", "hf_aligned_global_per_head"),
        layer_perhead_aggregation=p.get("layer_perhead_aggregation", "max"),
        allow_per_layer_mode=p.get("pruning_mode", "per_head") == "per_layer",
        disable_mlr=p.get("disable_mlr", False),
        disable_trig=p.get("disable_trig", False),
        protect_prefill=p.get("protect_prefill", False),
    )
    cfg.validate()
    return cfg


def gen_score_cases(ref_scoring, ref_config, out: dict):
    """Direct calls of compute_scores_pytorch on K.float() (scoring.py:207-362)."""
    gen = torch.Generator().manual_seed(synth.seed_for(90, 0))
    H, T, D = 4, 100, 128
    inv_freq = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(1, H, D, inv_freq, gen)
    fs = 0.5 + torch.rand((H, D // 2), generator=gen)
    offsets = torch.tensor([float(2 ** i) for i in range(17)])
    variants = [
        dict(aggregation="mean", disable_mlr=False, disable_trig=False, rope_style="half", round_start=100),
        dict(aggregation="max", disable_mlr=False, disable_trig=False, rope_style="half", round_start=100),
        dict(aggregation="mean", disable_mlr=True, disable_trig=False, rope_style="half", round_start=33000),
        dict(aggregation="mean", disable_mlr=False, disable_trig=True, rope_style="half", round_start=100),
        dict(aggregation="mean", disable_mlr=False, disable_trig=False, rope_style="interleaved", round_start=100001),
        dict(aggregation="max", disable_mlr=True, disable_trig=False, rope_style="interleaved", round_start=7),
    ]
    arrays = {
        "q_mean_real": stats.q_mean_real[0].numpy(),
        "q_mean_imag": stats.q_mean_imag[0].numpy(),
        "q_abs_mean": stats.q_abs_mean[0].numpy(),
        "freq_scale_sq": fs.numpy(),
        "omega": inv_freq.numpy(),
        "offsets": offsets.numpy(),
    }
    meta = []
    for i, v in enumerate(variants):
        k = synth.make_rotated_keys(H, T, D, inv_freq, gen, rope_style=v["rope_style"])  # [T,H,D]
        keys = k.permute(1, 0, 2).unsqueeze(0).contiguous()  # [1,H,T,D]
        cfg = ref_config.TriAttentionConfig(
            score_aggregation=v["aggregation"], disable_mlr=v["disable_mlr"], disable_trig=v["disable_trig"],
            rope_style=v["rope_style"], pruning_mode="per_head",
        )
        head_stats = {
            "q_mean_complex": torch.stack([stats.q_mean_real[0], stats.q_mean_imag[0]], dim=-1),
            "q_abs_mean": stats.q_abs_mean[0],
        }
        ref = ref_scoring.compute_scores_pytorch(
            key_states=keys.float(), cache_positions=None, head_stats=head_stats, omega=inv_freq,
            offsets=offsets, freq_scale_sq=fs, config=cfg, round_start=v["round_start"],
        )
        ref_bf16 = ref_scoring.compute_scores_pytorch(
            key_states=keys, cache_positions=None, head_stats=head_stats, omega=inv_freq,
            offsets=offsets, freq_scale_sq=fs, config=cfg, round_start=v["round_start"],
        )
        arrays[f"keys_{i}"] = bf16_to_np(keys)
        arrays[f"scores_{i}"] = ref.numpy()
        arrays[f"scores_bf16k_{i}"] = ref_bf16.float().numpy()
        meta.append(v)
    np.savez_compressed(HERE / "score_cases.npz", **arrays)
    out["score_cases"] = {"file": "score_cases.npz", "variants": meta, "shape": [1, H, T, D]}


def gen_selector_cases(out: dict):
    """Group selector + per-layer selectors + compaction through the reference's own runtime code."""
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.selector_hf import build_triattention_selector
    from triattention.vllm.runtime.kv_compaction import (
        compact_request_kv_in_place,
        compact_request_kv_in_place_per_head,
        register_kv_layout_axis_hint,
    )

    cases = {
        # tiny: inputs stored in the fixture
        "tiny_group": dict(seed=synth.seed_for(91, 0), num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=128,
                           theta=1e6, total_tokens=200, block_size=16, kv_axis=0, budget=64, window=16,
                           round_start=200, spare_blocks=2, store_inputs=True),
        # chunked (>4096 tokens), K/V axis 1, random block order
        "chunked_group": dict(seed=synth.seed_for(91, 1), num_layers=3, num_q_heads=8, num_kv_heads=2, head_dim=128,
                              theta=1e6, total_tokens=4500, block_size=16, kv_axis=1, budget=1024, window=128,
                              round_start=4500),
        # head shapes of the single-layer benchmark configuration, shorter, round_start != T, consecutive blocks (view fast path)
        "c0_like": dict(seed=synth.seed_for(91, 2), num_layers=1, num_q_heads=32, num_kv_heads=8, head_dim=128,
                        theta=1e6, total_tokens=2100, block_size=16, kv_axis=0, budget=512, window=128,
                        round_start=9000, consecutive_blocks=True),
        # llama3-scaled frequencies, ragged last block, no normalisation
        "llama3_nonorm": dict(seed=synth.seed_for(91, 3), num_layers=2, num_q_heads=8, num_kv_heads=4, head_dim=128,
                              theta=5e5, llama3=dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                     original_max_position_embeddings=8192),
                              total_tokens=1003, block_size=16, kv_axis=0, budget=256, window=32, round_start=20000,
                              normalize=False),
        # max over offsets, prefill protection
        "max_agg_prefill": dict(seed=synth.seed_for(91, 4), num_layers=2, num_q_heads=4, num_kv_heads=2, head_dim=128,
                                theta=1e6, total_tokens=700, block_size=16, kv_axis=0, budget=200, window=16,
                                round_start=700, aggregation="max", protect_prefill=True, prefill_len=40),
        # head_dim 64, group 8
        "d64_g8": dict(seed=synth.seed_for(91, 5), num_layers=2, num_q_heads=16, num_kv_heads=2, head_dim=64,
                       theta=1.5e5, total_tokens=900, block_size=16, kv_axis=1, budget=300, window=64,
                       round_start=1234),
        # legacy per-layer selection (z-norm -> group max -> guards -> top-k per layer)
        "legacy_layer_local": dict(seed=synth.seed_for(91, 6), num_layers=2, num_q_heads=8, num_kv_heads=2,
                                   head_dim=128, theta=1e6, total_tokens=640, block_size=16, kv_axis=0, budget=128,
                                   window=16, round_start=640, semantics="legacy_layer_local"),
        # shared keep set: max over heads (opt-in per_layer mode)
        "per_layer_shared": dict(seed=synth.seed_for(91, 7), num_layers=2, num_q_heads=8, num_kv_heads=2,
                                 head_dim=128, theta=1e6, total_tokens=640, block_size=16, kv_axis=0, budget=128,
                                 window=16, round_start=640, pruning_mode="per_layer"),
        # per_layer_per_head with mean over the GQA group
        "plph_mean": dict(seed=synth.seed_for(91, 8), num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=128,
                          theta=1e6, total_tokens=640, block_size=16, kv_axis=0, budget=128, window=16,
                          round_start=640, pruning_mode="per_layer_per_head", layer_perhead_aggregation="mean"),
    }
    arrays = {}
    with tempfile.TemporaryDirectory() as td:
        for name, p in cases.items():
            stats, caches, block_ids = build_paged_case(p)
            stats_path = Path(td) / f"{name}.pt"
            synth.save_stats_pt(stats, stats_path)
            cfg = runtime_config(ref_runtime_config, stats_path, p)
            sel_layer, sel_group, status = build_triattention_selector(cfg)
            assert status == "enabled", status
            for c in caches:
                if int(c.shape[0]) == 2 and int(c.shape[1]) == 2:
                    register_kv_layout_axis_hint(c, p["kv_axis"])
            T, bs = p["total_tokens"], p["block_size"]
            kw = dict(total_tokens=T, prefill_len=p.get("prefill_len", 0),
                      protect_prefill=p.get("protect_prefill", False), round_start=p["round_start"],
                      budget_total=min(p["budget"], T))
            p["input_sha256"] = sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches)
            p["block_ids"] = block_ids
            group_mode = (p.get("pruning_mode", "per_head") == "per_head"
                          and p.get("semantics", "hf_aligned_global_per_head") == "hf_aligned_global_per_head")
            if group_mode:
                def _iter():
                    for l, c in enumerate(caches):
                        yield l, c, block_ids, bs
                res = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, **kw)
                assert res["mode"] == "per_head"
                keep = res["indices"]
                arrays[f"{name}/keep"] = keep.numpy().astype(np.int32)
                keeps = [keep] * len(caches)
                modes = ["per_head"] * len(caches)
            else:
                keeps, modes = [], []
                for l, c in enumerate(caches):
                    res = sel_layer(keys_dense=None, kv_cache=c, block_ids=torch.as_tensor(block_ids),
                                    block_size=bs, layer_idx=l, **kw)
                    keeps.append(torch.as_tensor(res["indices"]))
                    modes.append(res["mode"])
                    arrays[f"{name}/keep_l{l}"] = keeps[-1].numpy().astype(np.int32)
            p["modes"] = modes
            # compaction through the reference (preserve_dropped_tokens=True, as layout_engine.py:71-80 forces)
            if p.get("store_inputs"):
                for l, c in enumerate(caches):
                    arrays[f"{name}/cache_in_l{l}"] = bf16_to_np(c)
                arrays[f"{name}/q_mean_real"] = stats.q_mean_real.numpy()
                arrays[f"{name}/q_mean_imag"] = stats.q_mean_imag.numpy()
                arrays[f"{name}/q_abs_mean"] = stats.q_abs_mean.numpy()
                arrays[f"{name}/inv_freq"] = stats.inv_freq.numpy()
            out_hashes = []
            for l, c in enumerate(caches):
                bt = torch.as_tensor(block_ids, dtype=torch.long)
                if modes[l] == "per_head":
                    n = compact_request_kv_in_place_per_head(
                        kv_cache=c, block_ids=bt, block_size=bs, keep_token_indices_per_head=keeps[l],
                        total_tokens=T, preserve_dropped_tokens=True)
                else:
                    n = compact_request_kv_in_place(
                        kv_cache=c, block_ids=bt, block_size=bs, keep_token_indices=keeps[l],
                        total_tokens=T, preserve_dropped_tokens=True)
                assert n == min(p["budget"], T)
                out_hashes.append(sha(c))
                if p.get("store_inputs"):
                    arrays[f"{name}/cache_out_l{l}"] = bf16_to_np(c)
            p["cache_out_sha256"] = out_hashes
    np.savez_compressed(HERE / "selector_cases.npz", **arrays)
    out["selector_cases"] = {"file": "selector_cases.npz", "cases": cases}


def gen_real_stats_case(out: dict):
    """Two layers of the shipped Qwen3-8B statistics as a non-synthetic stats source."""
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.selector_hf import build_triattention_selector

    src = REF / "triattention/calibration/for_aime25_experiment/qwen3_8b.pt"
    payload = torch.load(src, map_location="cpu", weights_only=False)
    L, H, D = 2, 32, 128
    qr = torch.stack([torch.stack([payload["stats"][f"layer{l:02d}_head{h:02d}"]["q_mean_real"] for h in range(H)])
                      for l in range(L)]).float()
    qi = torch.stack([torch.stack([payload["stats"][f"layer{l:02d}_head{h:02d}"]["q_mean_imag"] for h in range(H)])
                      for l in range(L)]).float()
    qa = torch.stack([torch.stack([payload["stats"][f"layer{l:02d}_head{h:02d}"]["q_abs_mean"] for h in range(H)])
                      for l in range(L)]).float()
    inv_freq = synth.rope_inv_freq(D, 1e6)
    stats = synth.SyntheticStats(qr, qi, qa, inv_freq, D, "half")
    p = dict(seed=synth.seed_for(92, 0), num_layers=L, num_q_heads=H, num_kv_heads=8, head_dim=D, theta=1e6,
             total_tokens=1500, block_size=16, kv_axis=0, budget=512, window=128, round_start=1500)
    gen = torch.Generator().manual_seed(p["seed"])
    T, bs = p["total_tokens"], p["block_size"]
    nblk = (T + bs - 1) // bs
    block_ids = synth.random_block_ids(nblk, nblk + 7, gen)
    caches = []
    for _l in range(L):
        cache = synth.make_paged_layer(nblk + 7, bs, 8, D, kv_axis=0)
        k = synth.make_rotated_keys(8, T, D, inv_freq, gen)
        v = synth.make_values(8, T, D, gen)
        synth.write_tokens_to_paged(cache, 0, block_ids, bs, k, v)
        caches.append(cache)
    with tempfile.TemporaryDirectory() as td:
        sp = Path(td) / "real.pt"
        synth.save_stats_pt(stats, sp)
        cfg = runtime_config(ref_runtime_config, sp, p)
        _, sel_group, status = build_triattention_selector(cfg)
        assert status == "enabled"

        def _iter():
            for l, c in enumerate(caches):
                yield l, c, block_ids, bs
        res = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, total_tokens=T,
                        prefill_len=0, protect_prefill=False, round_start=p["round_start"], budget_total=p["budget"])
    p["block_ids"] = block_ids
    p["input_sha256"] = sha(*caches)
    np.savez_compressed(
        HERE / "real_stats_case.npz",
        q_mean_real=qr.numpy(), q_mean_imag=qi.numpy(), q_abs_mean=qa.numpy(), inv_freq=inv_freq.numpy(),
        keep=res["indices"].numpy().astype(np.int32),
    )
    out["real_stats_case"] = {"file": "real_stats_case.npz", "params": p,
                              "source": "layers 0-1 of triattention/calibration/for_aime25_experiment/qwen3_8b.pt"}


def _reference_group_run(ref_runtime_config, build_triattention_selector, compact_fn, stats, caches, block_ids, p, td, tag):
    """Group selector + per-layer compaction of the reference on one request; returns (keep, output hashes)."""
    sp = Path(td) / f"{tag}.pt"
    synth.save_stats_pt(stats, sp)
    cfg = runtime_config(ref_runtime_config, sp, p)
    _, sel_group, status = build_triattention_selector(cfg)
    assert status == "enabled", status
    T, bs = p["total_tokens"], p["block_size"]

    def _iter():
        for l, c in enumerate(caches):
            yield l, c, block_ids, bs
    res = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, total_tokens=T, prefill_len=0,
                    protect_prefill=False, round_start=p["round_start"], budget_total=min(p["budget"], T))
    keep = res["indices"]
    hashes = []
    bt = torch.as_tensor(block_ids, dtype=torch.long)
    for c in caches:
        n = compact_fn(kv_cache=c, block_ids=bt, block_size=bs, keep_token_indices_per_head=keep, total_tokens=T,
                       preserve_dropped_tokens=True)
        assert n == min(p["budget"], T)
        hashes.append(sha(c))
    return keep, hashes


def gen_bench_shape_cases(out: dict):
    """The reference at the benchmark shapes: the single-layer configuration exactly (4096 tokens, budget 2048) and a
    one-request x two-layer slice at the benchmark length (32768 tokens).  Keep sets and output hashes only."""
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.selector_hf import build_triattention_selector
    from triattention.vllm.runtime.kv_compaction import compact_request_kv_in_place_per_head

    cases = {
        "c0_exact": dict(seed=synth.seed_for(94, 0), num_layers=1, num_q_heads=32, num_kv_heads=8, head_dim=128,
                         theta=1e6, total_tokens=4096, block_size=16, kv_axis=0, budget=2048, window=128,
                         round_start=4096),
        "c1_slice": dict(seed=synth.seed_for(94, 1), num_layers=2, num_q_heads=32, num_kv_heads=8, head_dim=128,
                         theta=1e6, total_tokens=32768, block_size=16, kv_axis=0, budget=2048, window=128,
                         round_start=32768),
    }
    arrays = {}
    with tempfile.TemporaryDirectory() as td:
        for name, p in cases.items():
            stats, caches, block_ids = build_paged_case(p)
            p["input_sha256"] = sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches)
            keep, hashes = _reference_group_run(ref_runtime_config, build_triattention_selector,
                                                compact_request_kv_in_place_per_head, stats, caches, block_ids, p, td, name)
            arrays[f"{name}/keep"] = keep.numpy().astype(np.int32)
            p["cache_out_sha256"] = hashes
    np.savez_compressed(HERE / "bench_shape_cases.npz", **arrays)
    out["bench_shape_cases"] = {"file": "bench_shape_cases.npz", "cases": cases}


def _stack_rkv(payload, layers, heads, key):
    return torch.stack([torch.stack([payload["stats"][f"layer{l:02d}_head{h:02d}"][key] for h in heads])
                        for l in layers]).float()


def gen_shipped_stats_cases(out: dict):
    """Shipped statistics as the stats source: all 36 layers of the Qwen3-8B file, and four layers of the head_dim-64
    GPT-OSS file with its YaRN frequencies (built by the installed transformers from the file's own rope_scaling)."""
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.selector_hf import build_triattention_selector
    from triattention.vllm.runtime.kv_compaction import compact_request_kv_in_place_per_head

    arrays, cases = {}, {}
    with tempfile.TemporaryDirectory() as td:
        # ---- Qwen3-8B, every layer
        payload = torch.load(REF / "triattention/calibration/for_aime24_experiment/qwen3_8b.pt", map_location="cpu",
                             weights_only=False)
        L, H, D = 36, 32, 128
        inv_freq = synth.rope_inv_freq(D, 1e6)
        stats = synth.SyntheticStats(_stack_rkv(payload, range(L), range(H), "q_mean_real"),
                                     _stack_rkv(payload, range(L), range(H), "q_mean_imag"),
                                     _stack_rkv(payload, range(L), range(H), "q_abs_mean"), inv_freq, D, "half")
        p = dict(seed=synth.seed_for(95, 0), num_layers=L, num_q_heads=H, num_kv_heads=8, head_dim=D, theta=1e6,
                 total_tokens=1200, block_size=16, kv_axis=0, budget=512, window=128, round_start=5000)
        _, caches, block_ids = build_paged_case(p)   # K/V and block ids from the seed; statistics from the file
        p["input_sha256"] = sha(*caches)
        keep, hashes = _reference_group_run(ref_runtime_config, build_triattention_selector,
                                            compact_request_kv_in_place_per_head, stats, caches, block_ids, p, td, "qwen3")
        arrays["qwen3_8b_all_layers/keep"] = keep.numpy().astype(np.int32)
        for k in ("q_mean_real", "q_mean_imag", "q_abs_mean"):
            arrays[f"qwen3_8b_all_layers/{k}"] = getattr(stats, k).numpy()
        p["cache_out_sha256_first_last"] = [hashes[0], hashes[-1]]
        p["source"] = "all 36 layers of triattention/calibration/for_aime24_experiment/qwen3_8b.pt"
        cases["qwen3_8b_all_layers"] = p

        # ---- GPT-OSS-120B statistics (head_dim 64, 64 query / 8 KV heads, YaRN)
        payload = torch.load(REF / "triattention/vllm/stats/gpt_oss_120b_stats.pt", map_location="cpu", weights_only=False)
        md = payload["metadata"]
        from transformers import LlamaConfig
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        rp = dict(md["rope_scaling"], rope_theta=float(md["rope_theta"]))
        yarn_inv, yarn_af = ROPE_INIT_FUNCTIONS["yarn"](
            LlamaConfig(hidden_size=64 * 64, num_attention_heads=64, head_dim=64, max_position_embeddings=131072,
                        rope_parameters=rp), "cpu")
        layers = [0, 11, 23, 35]
        L, H, D = len(layers), 64, 64
        stats = synth.SyntheticStats(_stack_rkv(payload, layers, range(H), "q_mean_real"),
                                     _stack_rkv(payload, layers, range(H), "q_mean_imag"),
                                     _stack_rkv(payload, layers, range(H), "q_abs_mean"), yarn_inv.float(), D, "half")
        p = dict(seed=synth.seed_for(95, 1), num_layers=L, num_q_heads=H, num_kv_heads=8, head_dim=D,
                 theta=float(md["rope_theta"]), total_tokens=900, block_size=16, kv_axis=0, budget=300, window=64,
                 round_start=2000)
        gen = torch.Generator().manual_seed(p["seed"])
        T, bs = p["total_tokens"], p["block_size"]
        nblk = (T + bs - 1) // bs
        block_ids = synth.random_block_ids(nblk, nblk + 5, gen)
        caches = []
        for _l in range(L):
            cache = synth.make_paged_layer(nblk + 5, bs, 8, D, kv_axis=0)
            synth.write_tokens_to_paged(cache, 0, block_ids, bs, synth.make_rotated_keys(8, T, D, stats.inv_freq, gen),
                                        synth.make_values(8, T, D, gen))
            caches.append(cache)
        p["input_sha256"] = sha(*caches)
        p["block_ids"] = block_ids
        keep, hashes = _reference_group_run(ref_runtime_config, build_triattention_selector,
                                            compact_request_kv_in_place_per_head, stats, caches, block_ids, p, td, "gptoss")
        arrays["gpt_oss_yarn/keep"] = keep.numpy().astype(np.int32)
        arrays["gpt_oss_yarn/inv_freq"] = stats.inv_freq.numpy()
        for k in ("q_mean_real", "q_mean_imag", "q_abs_mean"):
            arrays[f"gpt_oss_yarn/{k}"] = getattr(stats, k).numpy()
        p["cache_out_sha256"] = hashes
        p["layers"] = layers
        p["rope_scaling"] = {k: (float(v) if isinstance(v, (int, float)) and not isinstance(v, bool) else v)
                             for k, v in md["rope_scaling"].items()}
        p["attention_factor"] = float(yarn_af)
        p["source"] = "layers 0, 11, 23, 35 of triattention/vllm/stats/gpt_oss_120b_stats.pt"
        cases["gpt_oss_yarn"] = p
    np.savez_compressed(HERE / "shipped_stats_cases.npz", **arrays)
    out["shipped_stats_cases"] = {"file": "shipped_stats_cases.npz", "cases": cases}


SHIPPED_STATS = [
    "triattention/calibration/for_aime24_experiment/qwen3_8b.pt",
    "triattention/calibration/for_aime24_experiment/ds_llama8b.pt",
    "triattention/calibration/for_aime24_experiment/ds_qwen7b.pt",
    "triattention/calibration/for_aime25_experiment/qwen3_8b.pt",
    "triattention/calibration/for_aime25_experiment/ds_llama8b.pt",
    "triattention/calibration/for_aime25_experiment/ds_qwen7b.pt",
    "triattention/vllm/stats/gpt_oss_120b_stats.pt",
]


def gen_stats_loader_cases(out: dict):
    """What the reference's own loader (core/utils.py:18-134) returns for every statistics file it ships: metadata
    scalars and a hash of every per-layer tensor.  The Hub is unreachable here, so the loader's model-config
    fallbacks fail and it reports no inv_freq and freq_scale_sq = 1, which is what gets recorded."""
    from triattention.vllm.core.utils import load_frequency_stats

    files = {}
    for rel in SHIPPED_STATS:
        for nkv in (None, 8):
            try:
                md, hs = load_frequency_stats(REF / rel, device=torch.device("cpu"), dtype=torch.float32, num_kv_heads=nkv)
            except Exception as exc:  # a head count that 8 does not divide
                files[f"{rel}|kv={nkv}"] = {"error": type(exc).__name__}
                continue
            rec = {"metadata": {k: md[k] for k in ("num_attention_heads", "num_kv_heads", "head_dim", "num_layers",
                                                   "rope_style", "rope_type", "gqa_ratio") if k in md},
                   "rope_theta": float(md.get("rope_theta", 0.0)), "has_inv_freq": "inv_freq" in md,
                   "layers": sorted(int(l) for l in hs)}
            h = hashlib.sha256()
            for l in sorted(hs):
                for key in ("q_mean_complex", "q_abs_mean", "freq_scale_sq"):
                    h.update(hs[l][key].contiguous().numpy().tobytes())
            rec["tensors_sha256"] = h.hexdigest()
            files[f"{rel}|kv={nkv}"] = rec
    out["stats_loader_cases"] = {"files": files}


def gen_hook_cases(out: dict):
    """The reference's runner hook (hook_impl.py) driven on CPU with a fake runner: result dicts, block tables, caches."""
    import types
    import triattention.vllm.runtime.config as ref_runtime_config
    from triattention.vllm.runtime.hook_impl import make_runner_compression_hook
    from triattention.vllm.runtime.signals import CompressionSignal

    p = dict(seed=synth.seed_for(93, 0), num_layers=2, num_q_heads=8, num_kv_heads=2, head_dim=128, theta=1e6,
             total_tokens=900, block_size=16, kv_axis=0, budget=256, window=32, round_start=900)
    stats, caches, block_ids = build_paged_case(p)
    arrays, results = {}, {}
    with tempfile.TemporaryDirectory() as td:
        sp = Path(td) / "hook.pt"
        synth.save_stats_pt(stats, sp)
        cfg = runtime_config(ref_runtime_config, sp, p)
        T = p["total_tokens"]
        runner = types.SimpleNamespace(
            requests={"r0": types.SimpleNamespace(block_ids=(list(block_ids),), num_computed_tokens=T),
                      "r1": types.SimpleNamespace(block_ids=(list(block_ids[:8]),), num_computed_tokens=100)},
            kv_caches=caches, cache_config=types.SimpleNamespace(block_size=p["block_size"]))
        hook = make_runner_compression_hook(runner, cfg)
        so = types.SimpleNamespace(num_scheduled_tokens={"r0": 1, "r1": 1})

        def sig(req, est, **kw):
            base = dict(req_id=req, should_compress=True, reason="length_threshold", estimated_cache_len=est, step=1,
                        kv_usage=None, protect_prefill=False, prefill_len=0, scheduled_tokens=1)
            base.update(kw)
            return CompressionSignal(**base)

        results["under_budget"] = hook(req_id="r1", signal=sig("r1", 101), scheduler_output=so)
        results["not_found"] = hook(req_id="zz", signal=sig("zz", 500), scheduler_output=so)
        results["prefill_exceeds"] = hook(req_id="r0", signal=sig("r0", T + 1, protect_prefill=True, prefill_len=400),
                                          scheduler_output=so)
        results["compacted"] = hook(req_id="r0", signal=sig("r0", T + 1), scheduler_output=so)
        results["block_ids_after"] = [list(g) for g in runner.requests["r0"].block_ids]
        # the request grew by 40 tokens since: below budget + divide_length -> deferred
        runner.requests["r0"].num_computed_tokens = T + 40
        results["deferred"] = hook(req_id="r0", signal=sig("r0", 256 + 40 + 1), scheduler_output=so)
    p["block_ids"] = block_ids
    p["cache_out_sha256"] = [sha(c) for c in caches]
    out["hook_cases"] = {"params": p, "results": results}


def gen_input_patch_cases(out: dict):
    """Outputs of the reference's effective-length override helpers (runtime/input_patch_ops.py:66-215) on CPU tensors."""
    from triattention.vllm.runtime import input_patch_ops as ref

    gen = torch.Generator().manual_seed(20269001)
    arrays, cases = {}, {}

    def batch(num_reqs, num_rows, max_q, start=0, pad=0):
        rows = torch.randperm(num_rows, generator=gen)[:num_reqs].to(torch.int32)
        q_lens = torch.randint(0 if max_q > 1 else 1, max_q + 1, (num_reqs,), generator=gen)
        qsl = torch.zeros(num_reqs + 1, dtype=torch.int32)
        qsl[1:] = torch.cumsum(q_lens, 0).to(torch.int32)
        qsl += start
        total = int(qsl[-1]) + pad
        positions = torch.randint(0, 200000, (total,), generator=gen, dtype=torch.int64)
        seq_lens = torch.randint(1, 200000, (num_reqs + 3,), generator=gen, dtype=torch.int32)
        return rows, qsl, positions, seq_lens

    specs = {
        "decode_all_rows": dict(num_reqs=7, num_rows=16, max_q=1, frac=1.0),
        "mixed_prefill_sparse": dict(num_reqs=12, num_rows=40, max_q=9, frac=0.4),
        "single_request": dict(num_reqs=1, num_rows=4, max_q=5, frac=1.0),
        "offset_segments_padded": dict(num_reqs=6, num_rows=9, max_q=4, frac=0.5, start=3, pad=5),
        "missing_row": dict(num_reqs=5, num_rows=12, max_q=3, frac=0.6, extra_key=True),
        "zero_deltas_only": dict(num_reqs=4, num_rows=8, max_q=2, frac=0.5, zero_delta=True),
    }
    for name, sp in specs.items():
        rows, qsl, positions, seq_lens = batch(sp["num_reqs"], sp["num_rows"], sp["max_q"], sp.get("start", 0), sp.get("pad", 0))
        n_sel = max(1, int(round(sp["frac"] * sp["num_reqs"])))
        chosen = rows[torch.randperm(sp["num_reqs"], generator=gen)[:n_sel]].tolist()
        base_map = {int(r): int(torch.randint(1, 5000, (1,), generator=gen)) for r in chosen}
        delta_map = {int(r): (0 if sp.get("zero_delta") else -int(torch.randint(1, 3000, (1,), generator=gen))) for r in chosen}
        if sp.get("extra_key"):
            absent = [r for r in range(sp["num_rows"]) if r not in set(rows.tolist())][0]
            base_map[absent] = 77
            delta_map[absent] = -5
        dense = torch.randint(0, 9000, (sp["num_rows"],), generator=gen, dtype=torch.int32)
        s1 = seq_lens.clone()
        ref.overwrite_seq_lens_from_effective_lengths(idx_mapping=rows, query_start_loc=qsl,
                                                      effective_num_computed_tokens=dense, seq_lens=s1)
        s2 = seq_lens.clone()
        ok = ref.overwrite_seq_lens_from_effective_base_map(idx_mapping=rows, query_start_loc=qsl,
                                                            effective_base_by_req_idx=dict(base_map), seq_lens=s2)
        shifted = ref.shift_positions_from_sparse_deltas(idx_mapping=rows, query_start_loc=qsl, positions=positions,
                                                         pos_delta_by_req_idx=dict(delta_map))
        for k, v in dict(idx_mapping=rows, query_start_loc=qsl, positions=positions, seq_lens=seq_lens, dense_base=dense,
                         base_keys=torch.tensor(list(base_map.keys()), dtype=torch.int32),
                         base_vals=torch.tensor(list(base_map.values()), dtype=torch.int32),
                         delta_vals=torch.tensor([delta_map[k2] for k2 in base_map.keys()], dtype=torch.int32),
                         seq_lens_dense_out=s1, seq_lens_sparse_out=s2).items():
            arrays[f"{name}/{k}"] = v.numpy()
        if shifted is not None:
            arrays[f"{name}/positions_out"] = shifted.numpy()
        cases[name] = dict(sparse_applied=bool(ok), shifted=shifted is not None, num_rows=sp["num_rows"])
    np.savez_compressed(HERE / "input_patch_cases.npz", **arrays)
    out["input_patch_cases"] = {"file": "input_patch_cases.npz", "cases": cases}


def gen_calibration_cases(out: dict):
    """Statistics the reference's calibration arithmetic (scripts/calibrate.py:49-95, 223-240) derives from rotated queries."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_calibrate", str(REF / "scripts" / "calibrate.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    gen = torch.Generator().manual_seed(20269002)
    arrays, cases = {}, {}
    for name, (H, T, D, style, scale) in {"half_d128": (3, 37, 128, "half", 1.0),
                                          "interleaved_d64_scaled": (2, 20, 64, "interleaved", 0.5)}.items():
        inv = synth.rope_inv_freq(D, 1e6)
        pos = torch.arange(T, dtype=torch.float32)
        ang = pos[:, None] * inv[None, :]
        cosF, sinF = torch.cos(ang), torch.sin(ang)
        if style == "interleaved":
            cos = cosF.repeat_interleave(2, dim=-1)
            sin = sinF.repeat_interleave(2, dim=-1)
        else:
            cos = torch.cat((cosF, cosF), dim=-1)
            sin = torch.cat((sinF, sinF), dim=-1)
        q = torch.randn((1, H, T, D), generator=gen, dtype=torch.float32)
        q_rot = (q * cos[None, None] + ref._rotate_half(q, style=style) * sin[None, None]) * scale
        # the reference receives the model's rotary tables, which carry the attention scaling factor
        base = ref._invert_rope(q_rot, cos[None, None] * scale, sin[None, None] * scale, scale, style=style)
        mr, mi, ma = [], [], []
        for h in range(H):
            zc = ref._to_complex_pairs(base[0, h], style=style)
            m = zc.mean(dim=0)
            mr.append(m.real)
            mi.append(m.imag)
            ma.append(zc.abs().mean(dim=0))
        arrays[f"{name}/q_rot"] = q_rot.numpy()
        arrays[f"{name}/cos"] = cosF.numpy()
        arrays[f"{name}/sin"] = sinF.numpy()
        arrays[f"{name}/q_mean_real"] = torch.stack(mr).numpy()
        arrays[f"{name}/q_mean_imag"] = torch.stack(mi).numpy()
        arrays[f"{name}/q_abs_mean"] = torch.stack(ma).numpy()
        cases[name] = dict(rope_style=style, attn_scale=scale, head_dim=D)
    np.savez_compressed(HERE / "calibration_cases.npz", **arrays)
    out["calibration_cases"] = {"file": "calibration_cases.npz", "cases": cases}


def gen_runner_action_cases(out: dict):
    """Events, state-store calls and fatal errors of the reference's worker-side action driver
    (runtime/runner_compression_actions.py:11-237) on the scripted scenarios of tests/runner_action_scenarios.py."""
    from triattention.vllm.runtime.executor import CompressionExecutionResult
    from triattention.vllm.runtime.runner_compression_actions import execute_runner_compression_actions
    from triattention.vllm.runtime.signals import CompressionSignal
    import runner_action_scenarios as ras

    cases = {sc["name"]: ras.run_scenario(execute_runner_compression_actions, CompressionSignal,
                                          CompressionExecutionResult, sc) for sc in ras.scenarios()}
    (HERE / "runner_action_cases.json").write_text(json.dumps(cases, indent=1, sort_keys=True))
    out["runner_action_cases"] = {"file": "runner_action_cases.json", "cases": sorted(cases)}


def gen_state_store_cases(out: dict):
    """Snapshots of the reference's RequestStateStore (runtime/state.py:35-153) along tests/state_store_scenario.py."""
    from triattention.vllm.runtime.state import RequestStateStore
    import state_store_scenario as sss

    (HERE / "state_store_cases.json").write_text(json.dumps(sss.replay(RequestStateStore()), indent=1, sort_keys=True))
    out["state_store_cases"] = {"file": "state_store_cases.json", "calls": len(sss.CALLS)}


def gen_effective_override_cases(out: dict):
    """Results of the reference's build_effective_sparse_overrides (runtime/effective_overrides.py:209-359) on the
    scripted steps of tests/effective_override_scenarios.py."""
    from triattention.vllm.runtime.effective_overrides import build_effective_sparse_overrides
    import effective_override_scenarios as eos

    cases = {sc["name"]: eos.run_scenario(build_effective_sparse_overrides, sc) for sc in eos.scenarios()}
    (HERE / "effective_override_cases.json").write_text(json.dumps(cases, indent=1, sort_keys=True))
    out["effective_override_cases"] = {"file": "effective_override_cases.json", "cases": sorted(cases)}


def gen_step_lifecycle_cases(out: dict):
    """The reference's step life cycle (runtime/runner_state_updates.py + runner_compression_actions.py + state.py) along
    tests/step_lifecycle_scenario.py: events and store snapshots after every step."""
    import types
    from triattention.vllm.runtime import runner_compression_actions as rca, runner_state_updates as rsu
    from triattention.vllm.runtime.executor import CompressionExecutionResult
    from triattention.vllm.runtime.signals import CompressionSignal
    from triattention.vllm.runtime.state import RequestStateStore
    import step_lifecycle_scenario as sls

    mod = types.SimpleNamespace(
        register_new_requests=rsu.register_new_requests, cleanup_finished_requests=rsu.cleanup_finished_requests,
        mark_preemptions=rsu.mark_preemptions, mark_resumed=rsu.mark_resumed,
        consume_runner_signals=rsu.consume_runner_signals,
        execute_runner_compression_actions=rca.execute_runner_compression_actions)
    res = sls.replay(mod, RequestStateStore(), CompressionSignal, CompressionExecutionResult)
    (HERE / "step_lifecycle_cases.json").write_text(json.dumps(res, indent=1, sort_keys=True))
    out["step_lifecycle_cases"] = {"file": "step_lifecycle_cases.json", "steps": len(sls.STEPS)}


def gen_scheduler_side_cases(out: dict):
    """The reference's trigger planner (runtime/planner.py), effective-length tracker (effective_len_tracker.py),
    allocation-sync attributes (kv_allocation_sync.py) and block-pool reclaim (scheduler.py:29-52,338-564, called
    unbound on a stand-in scheduler) along tests/scheduler_side_scenarios.py.  Importing the scheduler module needs
    the serving engine the reference subclasses (installed in the build container)."""
    import types
    from triattention.vllm.runtime import kv_allocation_sync
    from triattention.vllm.runtime.effective_len_tracker import EffectiveCacheLenTracker
    from triattention.vllm.runtime.planner import CompressionPlanner
    from triattention.vllm.runtime.scheduler import TriAttentionScheduler
    import scheduler_side_scenarios as sss

    # the scheduler's step: the reference's patched schedule / update_from_output around stand-ins for the engine's own
    from triattention.vllm.runtime import integration_monkeypatch as im

    class _RefStepApi:
        @staticmethod
        def attach(sched, cfg):
            sched.triattention_config = cfg
            sched._planner = CompressionPlanner(cfg)
            sched._effective_len_tracker = EffectiveCacheLenTracker()
            sched._prefill_lens, sched._length_threshold_cache, sched._triattention_step = {}, {}, 0
            for name in ("_compute_length_threshold", "_resolve_prefill_len", "_has_active_effective_len_overrides"):
                setattr(sched, name, types.MethodType(getattr(TriAttentionScheduler, name), sched))

        @staticmethod
        def schedule(sched, base_schedule):
            im._ORIG_SCHED_SCHEDULE = base_schedule
            return im._patched_scheduler_schedule(sched)

        @staticmethod
        def update(sched, so, mro, base_update):
            im._ORIG_SCHED_UPDATE_FROM_OUTPUT = base_update
            return im._patched_scheduler_update_from_output(sched, so, mro)

    def ref_alloc(manager, request, num_new_tokens, *args, base_allocate, **kwargs):
        im._ORIG_KVCACHE_ALLOCATE_SLOTS = base_allocate
        return im._patched_kv_cache_allocate_slots(manager, request, num_new_tokens, *args, **kwargs)

    from triattention.vllm.runtime.signals import CompressionSignal

    res = {
        "alloc": {c["name"]: sss.run_alloc_case(ref_alloc, c) for c in sss.ALLOC_CASES},
        "boundary": sss.run_boundary_predicates(im._scheduler_output_has_compression_boundary,
                                                im._batch_queue_has_pending_compression_boundary, CompressionSignal),
        "steps": {name: sss.run_scheduler_steps(_RefStepApi, over) for name, over in sss.STEP_CONFIGS.items()},
        "planner": sss.replay_planner(CompressionPlanner),
        "tracker": sss.replay_tracker(EffectiveCacheLenTracker()),
        "allocation_sync": sss.replay_allocation_sync(kv_allocation_sync),
        "reclaim": {c["name"]: sss.run_reclaim_case(TriAttentionScheduler._apply_compression_events,
                                                    EffectiveCacheLenTracker, c) for c in sss.RECLAIM_CASES},
    }
    (HERE / "scheduler_side_cases.json").write_text(json.dumps(res, indent=1, sort_keys=True))
    out["scheduler_side_cases"] = {"file": "scheduler_side_cases.json", "reclaim_cases": sorted(res["reclaim"])}


def gen_worker_runner_cases(out: dict):
    """The reference's model-runner proxy (runtime/runner.py, runner_output_bridge.py, input_adapter.py) along
    tests/worker_runner_scenarios.py; methods that need no engine are called unbound on a stand-in."""
    import logging
    import types
    from triattention.vllm.runtime import input_adapter, runner_output_bridge
    from triattention.vllm.runtime.config import TriAttentionRuntimeConfig
    from triattention.vllm.runtime.runner import TriAttentionModelRunner as Ref
    from triattention.vllm.runtime.signals import CompressionSignal
    from triattention.vllm.runtime.state import RequestStateStore
    import worker_runner_scenarios as wrs

    log = logging.getLogger("ref_runner_scenarios")
    log.disabled = True

    def stand_in(base_runner, config, store, last_step=0):
        me = types.SimpleNamespace(config=config, state_store=store, _base_runner=base_runner, _logger=log,
                                   _last_step=last_step)
        me._get_actual_kv_from_block_table = types.MethodType(Ref._get_actual_kv_from_block_table, me)
        return me

    def self_trigger(base_runner, config, store, so, signals, last_step):
        return Ref._supplement_worker_self_triggers(stand_in(base_runner, config, store, last_step), so, signals)

    def trim(base_runner, store, so):
        Ref._patch_scheduler_output_for_compressed_reqs(stand_in(base_runner, None, store), so)

    def needs(store, so):
        return Ref._needs_effective_input_overrides(stand_in(None, None, store), so)

    cfg = TriAttentionRuntimeConfig(kv_budget=64, divide_length=16, protect_prefill=False, log_decisions=False,
                                    enable_experimental_kv_compaction=True)
    res = {
        "self_trigger": {c["name"]: wrs.run_self_trigger(self_trigger, RequestStateStore, c)
                         for c in wrs.self_trigger_cases(CompressionSignal)},
        "trim": {c["name"]: wrs.run_trim(trim, RequestStateStore, c) for c in wrs.TRIM_CASES},
        "overrides": {c["name"]: wrs.run_overrides(input_adapter.prepare_effective_input_overrides, needs,
                                                   RequestStateStore, c) for c in wrs.OVERRIDE_CASES},
        "attach": wrs.run_attach(runner_output_bridge),
        "steps": wrs.run_steps(Ref, cfg, CompressionSignal),
    }
    (HERE / "worker_runner_cases.json").write_text(json.dumps(res, indent=1, sort_keys=True))
    out["worker_runner_cases"] = {"file": "worker_runner_cases.json", "sections": sorted(res)}


def gen_input_patch_closure_cases(out: dict):
    """The reference's patched prepare_pos_seq_lens / compute_slot_mappings closures
    (runtime/input_patch_vllm_backend.py:105-244) with its own override state, on CPU tensors, along
    tests/input_patch_closure_scenarios.py."""
    from triattention.vllm.runtime import input_adapter, input_patch_state, input_patch_vllm_backend as be
    import input_patch_closure_scenarios as ipc

    class _RefApi:
        make_prepare = staticmethod(be.make_patched_prepare_pos_seq_lens)
        make_slots = staticmethod(be.make_patched_compute_slot_mappings)

        @staticmethod
        def scope(ov):
            return input_adapter.active_effective_input_overrides(input_adapter.EffectiveInputOverrides(**ov))

        @staticmethod
        def consumed():
            return input_patch_state.active_effective_overrides_consumed()

    res = {c["name"]: ipc.run_case(_RefApi, c, "cpu") for c in ipc.CASES}
    (HERE / "input_patch_closure_cases.json").write_text(json.dumps(res, indent=1, sort_keys=True))
    out["input_patch_closure_cases"] = {"file": "input_patch_closure_cases.json", "cases": sorted(res)}


PARTIAL = {
    # --only <name>: regenerate one group of fixtures and merge it into manifest.json
    "calibration": lambda out: gen_calibration_cases(out),
    "input_patch": lambda out: gen_input_patch_cases(out),
    "bench_shapes": lambda out: gen_bench_shape_cases(out),
    "shipped_stats": lambda out: gen_shipped_stats_cases(out),
    "stats_loader": lambda out: gen_stats_loader_cases(out),
    "runner_actions": lambda out: gen_runner_action_cases(out),
    "state_store": lambda out: gen_state_store_cases(out),
    "effective_overrides": lambda out: gen_effective_override_cases(out),
    "step_lifecycle": lambda out: gen_step_lifecycle_cases(out),
    "scheduler_side": lambda out: gen_scheduler_side_cases(out),
    "worker_runner": lambda out: gen_worker_runner_cases(out),
    "input_patch_closures": lambda out: gen_input_patch_closure_cases(out),
}


def main():
    if len(sys.argv) > 2 and sys.argv[1] == "--only":
        out = json.loads((HERE / "manifest.json").read_text())
        if sys.argv[2] in ("bench_shapes", "shipped_stats"):
            install_shims()
        PARTIAL[sys.argv[2]](out)
        (HERE / "manifest.json").write_text(json.dumps(out, indent=1, sort_keys=True))
        return
    ref_scoring, ref_config = install_shims()
    out = {"torch": torch.__version__}
    gen_score_cases(ref_scoring, ref_config, out)
    gen_selector_cases(out)
    gen_real_stats_case(out)
    gen_bench_shape_cases(out)
    gen_shipped_stats_cases(out)
    gen_stats_loader_cases(out)
    gen_hook_cases(out)
    gen_input_patch_cases(out)
    gen_calibration_cases(out)
    gen_runner_action_cases(out)
    gen_state_store_cases(out)
    gen_effective_override_cases(out)
    gen_step_lifecycle_cases(out)
    gen_scheduler_side_cases(out)
    gen_worker_runner_cases(out)
    gen_input_patch_closure_cases(out)
    (HERE / "manifest.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    print("wrote", [p.name for p in HERE.iterdir()])


if __name__ == "__main__":
    main()
