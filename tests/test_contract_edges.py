"""Edges of the reference contract that need no GPU: the legacy environment bridge, the request view over
the newer runner layout (block tables kept in batch arrays), rotary-frequency resolution for statistics files
that do not carry ``inv_freq``, and the fatal / soft split of compaction errors in the hook."""
from __future__ import annotations

import json
import types
import warnings

import numpy as np
import pytest
import torch

import oracle
import synth
from triattention_b200 import hook as hook_mod
from triattention_b200 import request_state, rope, selector as selector_mod, stats as stats_mod
from triattention_b200.config import TriAttentionRuntimeConfig, bridge_legacy_env
from triattention_b200.signals import CompressionSignal


# ------------------------------------------------------------------------------------------ legacy env bridge
def test_legacy_env_bridge():
    """TRIATTENTION_* -> TRIATTN_RUNTIME_* as the reference's plugin does it (plugin.py:37-58)."""
    env = {"TRIATTENTION_KV_BUDGET": "1024", "TRIATTENTION_DIVIDE_LENGTH": "64", "TRIATTENTION_WINDOW_SIZE": "32",
           "TRIATTENTION_LOG_DECISIONS": "0", "TRIATTENTION_STATS_PATH": "/tmp/s.pt",
           "TRIATTENTION_PRUNING_MODE": " Per_Layer_Head "}
    bridge_legacy_env(env)
    assert env["TRIATTN_RUNTIME_KV_BUDGET"] == "1024" and env["TRIATTN_RUNTIME_DIVIDE_LENGTH"] == "64"
    assert env["TRIATTN_RUNTIME_WINDOW_SIZE"] == "32" and env["TRIATTN_RUNTIME_LOG_DECISIONS"] == "0"
    assert env["TRIATTN_RUNTIME_SPARSE_STATS_PATH"] == "/tmp/s.pt"
    assert env["TRIATTN_RUNTIME_PRUNING_MODE"] == "per_layer_per_head"
    for name in ("ENABLE_EXPERIMENTAL_KV_COMPACTION", "ENABLE_EXPERIMENTAL_BLOCK_RECLAIM", "REQUIRE_TRITON_SCORING",
                 "REQUIRE_PHYSICAL_RECLAIM"):
        assert env["TRIATTN_RUNTIME_" + name] == "true"
    # a runtime variable that is already set wins; empty legacy values are ignored; explicit switches are kept
    env2 = {"TRIATTENTION_KV_BUDGET": "1024", "TRIATTN_RUNTIME_KV_BUDGET": "4096", "TRIATTENTION_WINDOW_SIZE": "",
            "TRIATTN_RUNTIME_REQUIRE_TRITON_SCORING": "false", "TRIATTN_RUNTIME_PRUNING_MODE": "per_head",
            "TRIATTENTION_PRUNING_MODE": "per_layer"}
    bridge_legacy_env(env2)
    assert env2["TRIATTN_RUNTIME_KV_BUDGET"] == "4096" and "TRIATTN_RUNTIME_WINDOW_SIZE" not in env2
    assert env2["TRIATTN_RUNTIME_REQUIRE_TRITON_SCORING"] == "false" and env2["TRIATTN_RUNTIME_PRUNING_MODE"] == "per_head"
    # an empty runtime variable does not block the legacy one
    env3 = {"TRIATTN_RUNTIME_KV_BUDGET": "", "TRIATTENTION_KV_BUDGET": "512"}
    bridge_legacy_env(env3)
    assert env3["TRIATTN_RUNTIME_KV_BUDGET"] == "512"


def test_legacy_env_bridge_feeds_from_env(monkeypatch):
    for k in ("TRIATTN_RUNTIME_KV_BUDGET", "TRIATTN_RUNTIME_PRUNING_MODE", "TRIATTN_RUNTIME_WINDOW_SIZE"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("TRIATTENTION_KV_BUDGET", "768")
    monkeypatch.setenv("TRIATTENTION_PRUNING_MODE", "per_layer_head")
    for k in ("ENABLE_EXPERIMENTAL_KV_COMPACTION", "ENABLE_EXPERIMENTAL_BLOCK_RECLAIM", "REQUIRE_TRITON_SCORING",
              "REQUIRE_PHYSICAL_RECLAIM"):
        monkeypatch.setenv("TRIATTN_RUNTIME_" + k, "true")   # registered with monkeypatch so they are undone
    bridge_legacy_env()
    cfg = TriAttentionRuntimeConfig.from_env()
    assert cfg.kv_budget == 768 and cfg.pruning_mode == "per_layer_per_head" and cfg.require_physical_reclaim
    monkeypatch.delenv("TRIATTN_RUNTIME_KV_BUDGET")
    monkeypatch.delenv("TRIATTN_RUNTIME_PRUNING_MODE")


# ------------------------------------------------------------------------------------------ batch-array request view
class _FakeBlockTables:
    """The slice of vLLM's block-table holder the request view touches (runner_struct_compat.py:84-135)."""

    def __init__(self, rows: int, width: int, groups: int = 1):
        self.block_tables = [types.SimpleNamespace(gpu=torch.zeros((rows, width), dtype=torch.int32))
                             for _ in range(groups)]
        self.num_blocks = types.SimpleNamespace(np=np.zeros((groups, rows), dtype=np.int32))
        self.staged, self.applied, self.calls = {}, 0, []

    def fill(self, gid, row, ids):
        self.block_tables[gid].gpu[row, : len(ids)] = torch.as_tensor(ids, dtype=torch.int32)
        self.num_blocks.np[gid, row] = len(ids)

    def append_block_ids(self, req_index, ids_by_group, overwrite=False):
        self.calls.append((req_index, tuple(list(g) for g in ids_by_group), overwrite))
        self.staged[req_index] = ids_by_group

    def apply_staged_writes(self):
        for row, groups in self.staged.items():
            for gid, ids in enumerate(groups):
                self.block_tables[gid].gpu[row].zero_()
                self.fill(gid, row, list(ids))
        self.staged.clear()
        self.applied += 1


def _batch_array_runner(ids_by_row, computed, width=64):
    bts = _FakeBlockTables(rows=len(ids_by_row), width=width)
    for row, ids in enumerate(ids_by_row):
        bts.fill(0, row, ids)
    req_ids = [f"r{i}" for i in range(len(ids_by_row))]
    return types.SimpleNamespace(
        block_tables=bts,
        req_states=types.SimpleNamespace(req_id_to_index={r: i for i, r in enumerate(req_ids)},
                                         num_computed_tokens=types.SimpleNamespace(
                                             gpu=torch.as_tensor(computed, dtype=torch.int32))),
        requests={r: types.SimpleNamespace(block_ids=([0],), num_computed_tokens=-1) for r in req_ids})


def test_compat_request_view_reads_and_rewrites_block_tables():
    runner = _batch_array_runner([[5, 9, 2, 7], [11, 3]], [60, 20])
    view, source = request_state.resolve_request_state_view(runner, "r1")
    assert source == "batch_arrays" and isinstance(view, request_state.CompatRequestStateView)
    assert view.req_index == 1 and view.num_computed_tokens == 20 and view.block_ids == ([11, 3],)
    v0, _ = request_state.resolve_request_state_view(runner, "r0")
    assert v0.block_ids == ([5, 9, 2, 7],) and v0.num_computed_tokens == 60
    # the setter is the block-table rewrite: staged with overwrite=True, applied, mirrored into requests[...]
    v0.block_ids = ([5, 9],)
    bts = runner.block_tables
    assert bts.calls == [(0, ([5, 9],), True)] and bts.applied == 1
    assert v0.block_ids == ([5, 9],) and runner.requests["r0"].block_ids == ([5, 9],)
    assert bts.block_tables[0].gpu[0, :4].tolist() == [5, 9, 0, 0] and int(bts.num_blocks.np[0, 0]) == 2
    with pytest.raises(TypeError):
        v0.block_ids = 7
    # rows without blocks fall back to the requests dictionary; unknown requests resolve to nothing
    bts.num_blocks.np[0, 1] = 0
    assert request_state.resolve_request_state_view(runner, "r1")[0].block_ids == ([0],)
    assert request_state.resolve_request_state_view(runner, "zz") == (None, "none")
    # the index can also come from input_batch.req_ids and the length from its host array
    runner2 = types.SimpleNamespace(
        block_tables=bts, input_batch=types.SimpleNamespace(req_ids=["r0", "r1"], num_computed_tokens_cpu=[60, 21]))
    v1, src = request_state.resolve_request_state_view(runner2, "r1")
    assert src == "batch_arrays" and v1.req_index == 1 and v1.num_computed_tokens == 21


def _recency_selector(heads):
    def build(config, base_runner=None):
        def group(*, layer_inputs=None, layer_input_iter=None, layer_kv_iter=None, total_tokens, prefill_len,
                  protect_prefill, round_start, budget_total):
            keep = torch.arange(total_tokens - budget_total, total_tokens).expand(heads, -1).contiguous()
            return {"mode": "per_head", "indices": keep, "semantic": "hf_aligned_global_per_head"}

        def layer(**kw):
            return None

        setattr(group, "_supports_paged_group", True)
        setattr(layer, "_supports_paged", True)
        return layer, group, "enabled"

    return build


def _small_case(T=200, bs=16, H=2, D=128, L=2, seed=5):
    gen = torch.Generator().manual_seed(seed)
    inv = synth.rope_inv_freq(D, 1e6)
    nblk = (T + bs - 1) // bs
    ids = synth.random_block_ids(nblk, nblk + 4, gen)
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(nblk + 4, bs, H, D, kv_axis=0)
        synth.write_tokens_to_paged(c, 0, ids, bs, synth.make_rotated_keys(H, T, D, inv, gen),
                                    synth.make_values(H, T, D, gen))
        caches.append(c)
    return caches, ids, inv


def test_hook_rewrites_block_table_through_batch_arrays(monkeypatch, tmp_path):
    """Hook -> compaction -> `req_state.block_ids = kept`: on the newer runner layout that assignment must land in
    block_tables.append_block_ids(overwrite=True) + apply_staged_writes() (runner_struct_compat.py:120-135)."""
    T, bs, budget = 200, 16, 64
    caches, ids, inv = _small_case(T, bs)
    before = [c.clone() for c in caches]
    runner = _batch_array_runner([ids], [T])
    runner.kv_caches = caches
    runner.cache_config = types.SimpleNamespace(block_size=bs)
    monkeypatch.setattr(hook_mod, "_build_triattention_selector", _recency_selector(2))
    monkeypatch.setattr(hook_mod, "compact_request_kv_in_place_per_head",
                        lambda kv_cache, block_ids, block_size, keep_token_indices_per_head, total_tokens,
                        preserve_dropped_tokens=True: oracle.compact_per_head(
                            kv_cache, block_ids.tolist(), block_size, keep_token_indices_per_head, total_tokens,
                            preserve_dropped_tokens, kv_axis=0))
    cfg = TriAttentionRuntimeConfig(kv_budget=budget, window_size=8, sparse_stats_path=tmp_path / "unused.pt")
    hook = hook_mod.make_runner_compression_hook(runner, cfg)
    sig = CompressionSignal("r0", True, "length_threshold", T + 1, 1, None, False, 0)
    out = hook(req_id="r0", signal=sig, scheduler_output=types.SimpleNamespace(num_scheduled_tokens={"r0": 1}))
    assert out["applied"] and out["cache_len_after"] == budget and out["reclaimed_block_count"] == len(ids) - budget // bs
    kept = ids[: budget // bs]
    bts = runner.block_tables
    assert bts.calls == [(0, (kept,), True)] and bts.applied == 1
    assert bts.block_tables[0].gpu[0, : len(ids)].tolist() == kept + [0] * (len(ids) - len(kept))
    assert out["block_reclaim"]["groups"][0]["block_ids_removed"] == ids[len(kept):]
    # kept tokens (the last `budget`) sit in slots 0..budget-1 of the kept blocks, K and V, every layer
    for c, b in zip(caches, before):
        flat_b = b[:, ids].reshape(2, -1, *b.shape[3:])[:, :T]
        flat_c = c[:, kept].reshape(2, -1, *c.shape[3:])[:, :budget]
        assert torch.equal(flat_c.view(torch.int16), flat_b[:, T - budget:].view(torch.int16))


def test_hook_inconsistent_layer_lengths_are_fatal(monkeypatch, tmp_path):
    """Layers that end at different lengths raise the fatal marker; any other compaction error is a soft failure
    (hook_group_pipeline.py:117-135)."""
    T, bs, budget = 200, 16, 64
    caches, ids, _ = _small_case(T, bs)
    runner = types.SimpleNamespace(requests={"r0": types.SimpleNamespace(block_ids=(list(ids),), num_computed_tokens=T)},
                                   kv_caches=caches, cache_config=types.SimpleNamespace(block_size=bs))
    monkeypatch.setattr(hook_mod, "_build_triattention_selector", _recency_selector(2))
    lens = iter([budget, budget - 1])
    monkeypatch.setattr(hook_mod, "compact_request_kv_in_place_per_head", lambda **kw: next(lens))
    cfg = TriAttentionRuntimeConfig(kv_budget=budget, window_size=8, sparse_stats_path=tmp_path / "unused.pt")
    sig = CompressionSignal("r0", True, "length_threshold", T + 1, 1, None, False, 0)
    so = types.SimpleNamespace(num_scheduled_tokens={"r0": 1})
    with pytest.raises(RuntimeError, match="TRIATTN_FATAL_TRITON_SCORING_REQUIRED:inconsistent_cache_len_after"):
        hook_mod.make_runner_compression_hook(runner, cfg)(req_id="r0", signal=sig, scheduler_output=so)

    def boom(**kw):
        raise IndexError("keep index out of range")

    monkeypatch.setattr(hook_mod, "compact_request_kv_in_place_per_head", boom)
    out = hook_mod.make_runner_compression_hook(runner, cfg)(req_id="r0", signal=sig, scheduler_output=so)
    assert out == {"applied": False, "reason": "compaction_failed:g0:l0:IndexError"}


# ------------------------------------------------------------------------------------------ rotary frequencies
def _bare_stats_file(path, L=2, H=8, D=128, model_name="Qwen/Qwen3-8B", extra=None):
    """A calibration file with exactly the metadata the reference's shipped files carry: no inv_freq, no rope_theta."""
    gen = torch.Generator().manual_seed(3)
    st = synth.make_stats(L, H, D, synth.rope_inv_freq(D, 1e6), gen)
    meta = {"rope_style": "half", "sampled_heads": [[l, h] for l in range(L) for h in range(H)], "head_dim": D,
            "model_name": model_name}
    meta.update(extra or {})
    recs = {f"layer{l:02d}_head{h:02d}": {"q_mean_real": st.q_mean_real[l, h].clone(), "q_mean_imag": st.q_mean_imag[l, h].clone(),
                                          "q_abs_mean": st.q_abs_mean[l, h].clone()} for l in range(L) for h in range(H)}
    torch.save({"metadata": meta, "stats": recs}, path)
    return st


def test_rope_formulas_match_transformers():
    tf = pytest.importorskip("transformers")
    try:
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    except Exception:
        pytest.skip("transformers without ROPE_INIT_FUNCTIONS")
    cases = [("llama3", 5e5, 128, dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                       original_max_position_embeddings=8192)),
             ("yarn", 150000.0, 64, dict(beta_fast=32.0, beta_slow=1.0, factor=32.0,
                                         original_max_position_embeddings=4096, truncate=False)),
             ("yarn", 1e6, 128, dict(factor=4.0, original_max_position_embeddings=32768)),
             ("linear", 1e4, 128, dict(factor=2.0))]
    for kind, theta, hd, params in cases:
        try:
            cfg = tf.LlamaConfig(hidden_size=hd * 4, num_attention_heads=4, head_dim=hd, max_position_embeddings=131072,
                                 rope_parameters=dict(params, rope_type=kind, rope_theta=theta))
            want, want_af = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
        except Exception:
            pytest.skip("this transformers build takes another config layout")
        got = rope.rope_spec_from_parameters(hd, theta, dict(params, rope_type=kind))
        assert torch.equal(got.inv_freq, want.float()), kind
        assert got.attention_factor == pytest.approx(float(want_af))
    plain = rope.rope_spec_from_parameters(128, 1e6)
    assert torch.equal(plain.inv_freq, stats_mod.compute_rope_frequencies(128, 1e6)) and plain.attention_factor == 1.0


def test_selector_state_resolves_rope_from_the_worker(tmp_path):
    """Shipped-style statistics (no inv_freq, no rope_theta) are scored with the served model's frequencies."""
    sp = tmp_path / "bare.pt"
    _bare_stats_file(sp)
    cfg = TriAttentionRuntimeConfig(sparse_stats_path=sp)
    qwen = torch.tensor([1e6 ** (-2.0 * f / 128) for f in range(64)], dtype=torch.float64)
    # (a) the runner's in-memory model config, older spelling
    runner = types.SimpleNamespace(model_config=types.SimpleNamespace(
        model="Qwen/Qwen3-8B", hf_config=types.SimpleNamespace(rope_theta=1e6, rope_scaling=None, head_dim=128,
                                                               hidden_size=4096, num_attention_heads=32)))
    st = selector_mod.load_scoring_state(sp, cfg, runner, strict=True)
    assert st["rope_source"] == "runner.model_config.hf_config"
    assert torch.equal(st["omega"], synth.rope_inv_freq(128, 1e6))
    assert torch.allclose(st["omega"].double(), qwen, rtol=1e-6)
    # (b) newer spelling: rope_parameters carries rope_theta; Llama-3.1 scaling
    l3 = dict(rope_type="llama3", rope_theta=5e5, factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
              original_max_position_embeddings=8192)
    runner_b = types.SimpleNamespace(vllm_config=types.SimpleNamespace(model_config=types.SimpleNamespace(
        model="x", hf_text_config={"rope_parameters": l3, "head_dim": 128})))
    st_b = selector_mod.load_scoring_state(sp, cfg, runner_b, strict=True)
    assert torch.equal(st_b["omega"], synth.rope_inv_freq(128, 5e5, l3))
    # (c) a local model directory named by the config wins over the runner object
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps({"rope_theta": 10000.0, "hidden_size": 1024, "num_attention_heads": 8,
                                                   "rope_scaling": {"type": "linear", "factor": 2.0}}))
    cfg_c = TriAttentionRuntimeConfig(sparse_stats_path=sp, model_path=mdir)
    st_c = selector_mod.load_scoring_state(sp, cfg_c, runner, strict=True)
    assert st_c["rope_source"].startswith("config.json:")
    assert torch.equal(st_c["omega"], stats_mod.compute_rope_frequencies(128, 10000.0) / 2.0)
    # (d) nothing names the frequencies: fatal when the native scorer is required, a warning otherwise
    with pytest.raises(RuntimeError, match="TRIATTN_FATAL_TRITON_SCORING_REQUIRED:rope_unresolved"):
        selector_mod.load_scoring_state(sp, cfg, None, strict=True)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        st_d = selector_mod.load_scoring_state(sp, cfg, None, strict=False)
    assert any("rope_theta=10000" in str(x.message) for x in w)
    assert torch.equal(st_d["omega"], stats_mod.compute_rope_frequencies(128, 10000.0))
    # (e) metadata inv_freq still has the last word
    sp2 = tmp_path / "with_inv.pt"
    inv = synth.rope_inv_freq(128, 12345.0)
    _bare_stats_file(sp2, extra={"inv_freq": inv})
    st_e = selector_mod.load_scoring_state(sp2, cfg, runner, strict=True)
    assert st_e["rope_source"] == "metadata.inv_freq" and torch.equal(st_e["omega"], inv)


def test_metadata_rope_scaling_sets_frequencies_and_scale(tmp_path):
    """Statistics that carry rope_theta + rope_scaling (YaRN, head_dim 64) resolve without any model config, and the
    rotary embedding's cos/sin factor lands in freq_scale_sq (core/utils.py:253-297)."""
    sp = tmp_path / "yarn.pt"
    yarn = {"beta_fast": 32.0, "beta_slow": 1.0, "factor": 32.0, "original_max_position_embeddings": 4096,
            "rope_type": "yarn", "truncate": False}
    _bare_stats_file(sp, L=1, H=4, D=64, model_name="openai/gpt-oss-120b",
                     extra={"rope_theta": 150000, "rope_type": "yarn", "rope_scaling": yarn})
    st = selector_mod.load_scoring_state(sp, TriAttentionRuntimeConfig(sparse_stats_path=sp), None, strict=True)
    want = rope.rope_spec_from_parameters(64, 150000.0, yarn)
    assert st["rope_source"] == "metadata.rope_theta" and torch.equal(st["omega"], want.inv_freq)
    af = 0.1 * float(np.log(32.0)) + 1.0
    assert st["attention_factor"] == pytest.approx(af)
    assert torch.allclose(st["head_stats"][0]["freq_scale_sq"], torch.full((4, 32), af * af))


# ------------------------------------------------------------------------------------------ perf line
def test_perf_profile_line(monkeypatch, tmp_path, caplog):
    """TRIATTN_RUNTIME_PERF_PROFILE: the hook is wrapped and a TRIATTN_PERF line is logged and written to the sink
    directory every TRIATTN_RUNTIME_PERF_LOG_EVERY calls (switches of runtime/perf_profile.py:54-62)."""
    import logging
    from triattention_b200.perf_profile import HookPerfProfile
    calls = []

    def hook(req_id, signal, scheduler_output):
        calls.append(req_id)
        if req_id == "boom":
            raise RuntimeError("x")
        return {"applied": req_id == "a", "reason": "kv_compacted:per_head" if req_id == "a" else "under_budget"}

    assert HookPerfProfile.from_env().wrap(hook) is hook          # both switches off: the hook itself
    monkeypatch.setenv("TRIATTN_RUNTIME_PERF_PROFILE", "1")
    monkeypatch.setenv("TRIATTN_RUNTIME_PERF_LOG_EVERY", "3")
    monkeypatch.setenv("TRIATTN_RUNTIME_PERF_SINK_DIR", str(tmp_path))
    prof = HookPerfProfile.from_env(logging.getLogger("perf_test"))
    wrapped = prof.wrap(hook)
    with caplog.at_level(logging.INFO, logger="perf_test"):
        assert wrapped("a", None, None)["applied"]
        assert wrapped("b", None, None)["reason"] == "under_budget"
        with pytest.raises(RuntimeError):
            wrapped("boom", None, None)
    assert (prof.calls, prof.applied, prof.skipped, prof.errors) == (3, 1, 1, 1)
    line = prof.summary_line()
    assert line.startswith("TRIATTN_PERF steps=3 ") and "applied=1 skipped=1 errors=1" in line
    assert "top_skip_reasons=under_budget:1" in line and "avg_ms(compress=" in line
    assert any("TRIATTN_PERF" in r.getMessage() for r in caplog.records)
    sink = list(tmp_path.glob("triattn_perf_*.log"))
    assert len(sink) == 1 and sink[0].read_text().startswith("TRIATTN_PERF steps=3")
