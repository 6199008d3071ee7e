"""Host-side mirror of the reference interface, on CPU: config, stats loader, hook orchestration.

The hook is driven with the CPU checker injected as selector / compaction (the seams the reference itself
exposes for fake-runner tests) and compared with result dicts produced by the reference's own hook.
"""
from __future__ import annotations

import types
from pathlib import Path

import pytest
import torch

import oracle
from conftest import tensor_sha
from golden_cases import build_paged_case, stats_by_layer
from triattention_b200 import hook as hook_mod
from triattention_b200 import kv_compaction, stats as stats_mod
import synth
from triattention_b200.config import TriAttentionConfig, TriAttentionRuntimeConfig
from triattention_b200.plan_models import KeepPlan
from triattention_b200.signals import CompressionSignal


def test_runtime_config_env(monkeypatch):
    for k in ("KV_BUDGET", "WINDOW_SIZE", "PROTECT_PREFILL", "SPARSE_STATS_PATH", "PRUNING_MODE", "KV_USAGE_TRIGGER"):
        monkeypatch.delenv("TRIATTN_RUNTIME_" + k, raising=False)
    d = TriAttentionRuntimeConfig.from_env()
    assert (d.kv_budget, d.divide_length, d.window_size, d.pruning_mode) == (2048, 128, 128, "per_head")
    assert d.sparse_score_aggregation == "mean" and d.sparse_normalize_scores and d.require_triton_scoring
    assert d.per_head_selection_semantics == "hf_aligned_global_per_head" and d.score_chunk_max_tokens == 4096
    monkeypatch.setenv("TRIATTN_RUNTIME_KV_BUDGET", "1024")
    monkeypatch.setenv("TRIATTN_RUNTIME_PROTECT_PREFILL", "yes")
    monkeypatch.setenv("TRIATTN_RUNTIME_SPARSE_STATS_PATH", " /tmp/x.pt ")
    monkeypatch.setenv("TRIATTN_RUNTIME_KV_USAGE_TRIGGER", "0.95")
    c = TriAttentionRuntimeConfig.from_env()
    assert c.kv_budget == 1024 and c.protect_prefill is True and c.sparse_stats_path == Path("/tmp/x.pt")
    assert c.kv_usage_trigger == 0.95
    monkeypatch.setenv("TRIATTN_RUNTIME_PROTECT_PREFILL", "maybe")
    with pytest.raises(ValueError, match="Invalid boolean"):
        TriAttentionRuntimeConfig.from_env()
    monkeypatch.setenv("TRIATTN_RUNTIME_PROTECT_PREFILL", "0")
    monkeypatch.setenv("TRIATTN_RUNTIME_PRUNING_MODE", "per_layer")
    with pytest.raises(ValueError, match="disabled by default"):
        TriAttentionRuntimeConfig.from_env()
    with pytest.raises(ValueError, match="kv_budget must be > 0"):
        TriAttentionRuntimeConfig(kv_budget=0).validate()
    with pytest.raises(ValueError, match="hysteresis"):
        TriAttentionRuntimeConfig(kv_usage_release=0.99).validate()
    with pytest.raises(ValueError, match="window_size"):
        TriAttentionConfig(kv_budget=64, window_size=64)
    assert TriAttentionConfig(pruning_mode="per_layer_per_head").pruning_mode == "per_head"


def test_stats_loader_both_formats(tmp_path):
    gen = torch.Generator().manual_seed(1)
    inv = synth.rope_inv_freq(128, 1e6)
    st = synth.make_stats(3, 8, 128, inv, gen)
    p = tmp_path / "rkv.pt"
    synth.save_stats_pt(st, p)
    meta, hs = stats_mod.load_frequency_stats(p)
    assert meta["num_layers"] == 3 and meta["num_attention_heads"] == 8 and meta["head_dim"] == 128
    assert torch.equal(meta["inv_freq"], inv)
    assert torch.equal(hs[1]["q_mean_complex"][..., 0], st.q_mean_real[1])
    assert torch.equal(hs[2]["q_abs_mean"], st.q_abs_mean[2])
    assert torch.equal(hs[0]["freq_scale_sq"], torch.ones(8, 64))
    # GQA mean when the caller asks for KV-head statistics
    meta2, hs2 = stats_mod.load_frequency_stats(p, num_kv_heads=2)
    assert meta2["gqa_ratio"] == 4
    assert torch.allclose(hs2[0]["q_abs_mean"], st.q_abs_mean[0].reshape(2, 4, 64).mean(1))
    # native format
    native = {"metadata": {"num_attention_heads": 8, "num_kv_heads": 8, "head_dim": 128, "num_layers": 1,
                           "rope_theta": 10000.0},
              "layer_stats": {0: {"q_mean_complex": torch.randn(8, 64, 2), "freq_scale_sq": torch.ones(8, 64)}}}
    p2 = tmp_path / "native.pt"
    torch.save(native, p2)
    meta3, hs3 = stats_mod.load_frequency_stats(p2)
    assert hs3[0]["q_mean_complex"].shape == (8, 64, 2)
    assert torch.allclose(stats_mod.resolve_omega(meta3, 128), stats_mod.compute_rope_frequencies(128, 10000.0))
    with pytest.raises(FileNotFoundError):
        stats_mod.load_frequency_stats(tmp_path / "missing.pt")
    torch.save({"metadata": {}, "layer_stats": {}}, tmp_path / "bad.pt")
    with pytest.raises(ValueError, match="missing required metadata"):
        stats_mod.load_frequency_stats(tmp_path / "bad.pt")
    assert stats_mod.geometric_offsets(65536).tolist() == [float(2 ** i) for i in range(17)]
    assert stats_mod.resolve_layer_for_stats(5, (0, 1, 2)) == 2 and stats_mod.resolve_layer_for_stats(1, (0, 1, 2)) == 1


def test_keep_plan_and_fallback_keep():
    assert KeepPlan.from_selector_result({"mode": "per_head", "indices": torch.zeros(2, 5)}).keep_count() == 5
    assert KeepPlan.from_selector_result({"indices": [1, 2, 3]}).keep_count() == 3
    plan = KeepPlan("per_head", [[1, 2], [3, 4]], "hf_aligned_global_per_head")
    assert plan.selection_mode_label == "per_head:hf_aligned_global_per_head" and plan.keep_count() == 2
    with pytest.raises(ValueError):
        KeepPlan("per_head", torch.zeros(5)).keep_count()
    for args in [(10, 4, 0, False), (10, 4, 2, True), (10, 4, 5, True), (3, 4, 0, False), (10, 4, 5, True, False)]:
        assert kv_compaction.build_keep_token_indices(*args) == oracle.fallback_keep_indices(*args)


def _oracle_selector_builder(p, stats, caches):
    """Selector callables with the reference signature, computed by the CPU checker."""
    sl = stats_by_layer(stats)

    def build(config, base_runner=None):
        def group(*, layer_inputs=None, layer_input_iter=None, layer_kv_iter=None, total_tokens, prefill_len,
                  protect_prefill, round_start, budget_total):
            layers = list(layer_kv_iter())
            if total_tokens <= budget_total:
                return {"mode": "per_head", "indices": torch.arange(total_tokens).expand(2, -1).contiguous()}
            if protect_prefill and config.include_prefill_in_budget and prefill_len > budget_total:
                return None
            keep = oracle.select_group_per_head(layers, sl, stats.inv_freq, oracle.geometric_offsets(), total_tokens,
                                                round_start, budget_total, window_size=config.window_size,
                                                prefill_len=prefill_len, protect_prefill=protect_prefill, kv_axis=0)
            return {"mode": "per_head", "indices": keep, "semantic": "hf_aligned_global_per_head"}

        def layer(**kw):
            return None

        setattr(group, "_supports_paged_group", True)
        setattr(layer, "_supports_paged", True)
        return layer, group, "enabled"

    return build


def test_hook_orchestration_matches_reference_hook(manifest, monkeypatch, tmp_path):
    hc = manifest["hook_cases"]
    p, want = hc["params"], hc["results"]
    stats, caches, block_ids = build_paged_case(p)
    assert block_ids == p["block_ids"]
    monkeypatch.setattr(hook_mod, "_build_triattention_selector", _oracle_selector_builder(p, stats, caches))
    monkeypatch.setattr(hook_mod, "compact_request_kv_in_place_per_head",
                        lambda kv_cache, block_ids, block_size, keep_token_indices_per_head, total_tokens,
                        preserve_dropped_tokens=True: oracle.compact_per_head(
                            kv_cache, block_ids.tolist(), block_size, keep_token_indices_per_head, total_tokens,
                            preserve_dropped_tokens, kv_axis=0))
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    cfg = TriAttentionRuntimeConfig(kv_budget=p["budget"], window_size=p["window"], sparse_stats_path=sp,
                                    preserve_dropped_tokens=True)
    T = p["total_tokens"]
    runner = types.SimpleNamespace(
        requests={"r0": types.SimpleNamespace(block_ids=(list(block_ids),), num_computed_tokens=T),
                  "r1": types.SimpleNamespace(block_ids=(list(block_ids[:8]),), num_computed_tokens=100)},
        kv_caches=caches, cache_config=types.SimpleNamespace(block_size=p["block_size"]))
    hook_mod.install_runner_compression_hook(runner, cfg)
    hook = runner.triattention_apply_compression
    so = types.SimpleNamespace(num_scheduled_tokens={"r0": 1, "r1": 1})

    def sig(req, est, **kw):
        base = dict(req_id=req, should_compress=True, reason="length_threshold", estimated_cache_len=est, step=1,
                    kv_usage=None, protect_prefill=False, prefill_len=0, scheduled_tokens=1)
        base.update(kw)
        return CompressionSignal(**base)

    assert hook(req_id="r1", signal=sig("r1", 101), scheduler_output=so) == want["under_budget"]
    assert hook(req_id="zz", signal=sig("zz", 500), scheduler_output=so) == want["not_found"]
    assert hook(req_id="r0", signal=sig("r0", T + 1, protect_prefill=True, prefill_len=400),
                scheduler_output=so) == want["prefill_exceeds"]
    got = hook(req_id="r0", signal=sig("r0", T + 1), scheduler_output=so)
    assert got == want["compacted"]
    assert [list(g) for g in runner.requests["r0"].block_ids] == want["block_ids_after"]
    assert [tensor_sha(c) for c in caches] == p["cache_out_sha256"]
    runner.requests["r0"].num_computed_tokens = T + 40
    assert hook(req_id="r0", signal=sig("r0", 256 + 40 + 1), scheduler_output=so) == want["deferred"]
    assert runner._triattention_active_req_id == "r0"
    # a second install keeps the existing hook
    hook_mod.install_runner_compression_hook(runner, cfg)
    assert runner.triattention_apply_compression is hook


def test_hook_soft_failures(monkeypatch, tmp_path):
    gen = torch.Generator().manual_seed(2)
    st = synth.make_stats(1, 2, 128, synth.rope_inv_freq(128, 1e6), gen)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(st, sp)
    monkeypatch.setattr(hook_mod, "_build_triattention_selector", lambda config, base_runner=None: (None, None, "stats_path_not_set"))
    cfg = TriAttentionRuntimeConfig(kv_budget=8, window_size=2, sparse_stats_path=sp, require_triton_scoring=False)
    sig = CompressionSignal("r", True, "length_threshold", 101, 1, None, False, 0)
    so = types.SimpleNamespace(num_scheduled_tokens={"r": 1})
    req = types.SimpleNamespace(block_ids=(list(range(1, 121)),), num_computed_tokens=100)
    r1 = types.SimpleNamespace(requests={"r": req}, kv_caches=None, cache_config=None)
    assert hook_mod.make_runner_compression_hook(r1, cfg)("r", sig, so)["reason"] == "kv_cache_unavailable"
    r2 = types.SimpleNamespace(requests={"r": req}, kv_caches=[], cache_config=types.SimpleNamespace(block_size=0))
    assert hook_mod.make_runner_compression_hook(r2, cfg)("r", sig, so)["reason"] == "invalid_block_size"
    r3 = types.SimpleNamespace(requests={"r": types.SimpleNamespace(block_ids=None, num_computed_tokens=100)},
                               kv_caches=[], cache_config=types.SimpleNamespace(block_size=16))
    assert hook_mod.make_runner_compression_hook(r3, cfg)("r", sig, so)["reason"] == "missing_block_ids"
    r4 = types.SimpleNamespace(requests={"r": req}, kv_caches=[], cache_config=types.SimpleNamespace(block_size=16))
    assert hook_mod.make_runner_compression_hook(r4, cfg)("r", sig, so)["reason"] == "no_compactable_groups"
    plan_cfg = TriAttentionRuntimeConfig(kv_budget=8, window_size=2, sparse_stats_path=sp,
                                         enable_experimental_kv_compaction=False, require_physical_reclaim=False)
    out = hook_mod.make_runner_compression_hook(r4, plan_cfg)("r", sig, so)
    assert out == {"applied": False, "reason": "plan_only", "cache_len_after": 8}
    # strict mode: a missing selector is fatal and carries the reference's marker
    strict_cfg = TriAttentionRuntimeConfig(kv_budget=8, window_size=2, sparse_stats_path=sp)
    with pytest.raises(RuntimeError, match="TRIATTN_FATAL_TRITON_SCORING_REQUIRED:selector_unavailable"):
        hook_mod.make_runner_compression_hook(r4, strict_cfg)("r", sig, so)
