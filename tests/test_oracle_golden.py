"""The CPU checker (oracle/) replayed against outputs of the reference itself (tests/golden/)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from conftest import np_to_bf16, tensor_sha
from golden_cases import build_paged_case, build_real_stats_case, stats_by_layer


def test_offsets():
    off = oracle.geometric_offsets(65536)
    assert off.tolist() == [float(2 ** i) for i in range(17)]
    with pytest.raises(ValueError):
        oracle.geometric_offsets(0)


def test_score_cases_match_reference(manifest, score_cases):
    info = manifest["score_cases"]
    a = score_cases
    for i, v in enumerate(info["variants"]):
        keys = np_to_bf16(a[f"keys_{i}"])
        got = oracle.score_keys_reference(
            keys, torch.from_numpy(a["q_mean_real"]), torch.from_numpy(a["q_mean_imag"]),
            torch.from_numpy(a["q_abs_mean"]), torch.from_numpy(a["freq_scale_sq"]),
            torch.from_numpy(a["omega"]), torch.from_numpy(a["offsets"]), v["round_start"],
            aggregation=v["aggregation"], disable_mlr=v["disable_mlr"], disable_trig=v["disable_trig"],
            rope_style=v["rope_style"])
        ref = torch.from_numpy(a[f"scores_{i}"])
        # same torch ops in the same order: bit-identical
        assert torch.equal(got, ref), f"variant {i}: max diff {(got - ref).abs().max()}"
        # exact-arithmetic checker agrees with the fp32 reference far inside the 1e-3 contract
        ex = oracle.score_keys_exact64(
            keys, torch.from_numpy(a["q_mean_real"]), torch.from_numpy(a["q_mean_imag"]),
            torch.from_numpy(a["q_abs_mean"]), torch.from_numpy(a["freq_scale_sq"]),
            torch.from_numpy(a["omega"]), torch.from_numpy(a["offsets"]), v["round_start"],
            aggregation=v["aggregation"], disable_mlr=v["disable_mlr"], disable_trig=v["disable_trig"],
            rope_style=v["rope_style"])
        scale = max(float(ref.abs().max()), 1.0)
        assert np.abs(ex - ref.numpy().astype(np.float64)).max() / scale < 2e-5


def _case_kwargs(p):
    return dict(
        window_size=p["window"], prefill_len=p.get("prefill_len", 0), protect_prefill=p.get("protect_prefill", False),
        normalize=p.get("normalize", True), aggregation=p.get("aggregation", "mean"),
        disable_mlr=p.get("disable_mlr", False), disable_trig=p.get("disable_trig", False),
        rope_style=p.get("rope_style", "half"), kv_axis=p["kv_axis"],
    )


GROUP_CASES = ["tiny_group", "chunked_group", "c0_like", "llama3_nonorm", "max_agg_prefill", "d64_g8"]


@pytest.mark.parametrize("name", GROUP_CASES)
def test_group_selector_and_compaction_match_reference(manifest, selector_cases, name):
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    assert block_ids == p["block_ids"]
    assert tensor_sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches) == p["input_sha256"], \
        "seeded inputs differ from the ones the fixture was generated with"
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    offsets = oracle.geometric_offsets()
    keep = oracle.select_group_per_head(
        layers, stats_by_layer(stats), stats.inv_freq, offsets, T, p["round_start"], min(p["budget"], T),
        **_case_kwargs(p))
    ref_keep = torch.from_numpy(selector_cases[f"{name}/keep"]).long()
    assert torch.equal(keep, ref_keep)
    for l, c in enumerate(caches):
        n = oracle.compact_per_head(c, block_ids, bs, keep, T, preserve_dropped_tokens=True, kv_axis=p["kv_axis"])
        assert n == keep.shape[1]
        assert tensor_sha(c) == p["cache_out_sha256"][l]


def test_tiny_case_stored_inputs(manifest, selector_cases):
    """The tiny fixture also carries its inputs/outputs verbatim, independent of the generator."""
    p = manifest["selector_cases"]["cases"]["tiny_group"]
    a = selector_cases
    caches = [np_to_bf16(a[f"tiny_group/cache_in_l{l}"]).clone() for l in range(p["num_layers"])]
    stats = {
        l: {
            "q_mean_real": torch.from_numpy(a["tiny_group/q_mean_real"][l]),
            "q_mean_imag": torch.from_numpy(a["tiny_group/q_mean_imag"][l]),
            "q_abs_mean": torch.from_numpy(a["tiny_group/q_abs_mean"][l]),
            "freq_scale_sq": torch.ones(p["num_q_heads"], p["head_dim"] // 2),
        }
        for l in range(p["num_layers"])
    }
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, p["block_ids"], bs) for l, c in enumerate(caches)]
    keep = oracle.select_group_per_head(
        layers, stats, torch.from_numpy(a["tiny_group/inv_freq"]), oracle.geometric_offsets(), T,
        p["round_start"], p["budget"], **_case_kwargs(p))
    assert torch.equal(keep, torch.from_numpy(a["tiny_group/keep"]).long())
    for l, c in enumerate(caches):
        oracle.compact_per_head(c, p["block_ids"], bs, keep, T, kv_axis=p["kv_axis"])
        assert torch.equal(c.view(torch.int16), np_to_bf16(a[f"tiny_group/cache_out_l{l}"]).view(torch.int16))


@pytest.mark.parametrize("name,mode,group_agg,reduce_stats", [
    ("legacy_layer_local", "per_head", "max", True),
    ("per_layer_shared", "shared", "max", True),
    ("plph_mean", "per_head", "mean", False),
])
def test_layer_local_selectors_match_reference(manifest, selector_cases, name, mode, group_agg, reduce_stats):
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    assert tensor_sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches) == p["input_sha256"]
    T, bs = p["total_tokens"], p["block_size"]
    sl = stats_by_layer(stats)
    kw = _case_kwargs(p)
    for l, c in enumerate(caches):
        keep = oracle.select_layer_local(
            c, block_ids, bs, sl[l], stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"],
            p["budget"], mode=mode, group_agg=group_agg, reduce_stats=reduce_stats, **kw)
        ref_keep = torch.from_numpy(selector_cases[f"{name}/keep_l{l}"]).long()
        assert p["modes"][l] == mode
        assert torch.equal(keep, ref_keep)
        if mode == "shared":
            oracle.compact_shared(c, block_ids, bs, keep, T, kv_axis=p["kv_axis"])
        else:
            oracle.compact_per_head(c, block_ids, bs, keep, T, kv_axis=p["kv_axis"])
        assert tensor_sha(c) == p["cache_out_sha256"][l]


def test_real_stats_case(manifest, real_stats_case):
    p = manifest["real_stats_case"]["params"]
    stats, caches, block_ids = build_real_stats_case(p, real_stats_case)
    assert block_ids == p["block_ids"]
    assert tensor_sha(*caches) == p["input_sha256"]
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    keep = oracle.select_group_per_head(
        layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"],
        p["budget"], window_size=p["window"], kv_axis=0)
    assert torch.equal(keep, torch.from_numpy(real_stats_case["keep"]).long())


def test_prefix_only_compaction_is_prefix_of_full():
    """preserve_dropped_tokens=False writes exactly the kept prefix and nothing else."""
    g = torch.Generator().manual_seed(5)
    T, bs, H, D = 70, 16, 3, 8
    cache = torch.randn((2, 9, bs, H, D), generator=g).to(torch.bfloat16)
    block_ids = [7, 1, 4, 2, 8]
    keep = torch.stack([torch.sort(torch.randperm(T, generator=g)[:20]).values for _ in range(H)])
    a, b = cache.clone(), cache.clone()
    oracle.compact_per_head(a, block_ids, bs, keep, T, preserve_dropped_tokens=True)
    oracle.compact_per_head(b, block_ids, bs, keep, T, preserve_dropped_tokens=False)
    ka = oracle.gather_request_k_dense(a, block_ids, bs, T)
    kb = oracle.gather_request_k_dense(b, block_ids, bs, T)
    k0 = oracle.gather_request_k_dense(cache, block_ids, bs, T)
    assert torch.equal(ka[:, :, :20], kb[:, :, :20])
    assert torch.equal(kb[:, :, 20:], k0[:, :, 20:])
    for h in range(H):
        assert torch.equal(kb[0, h, :20], k0[0, h, keep[h]])


def test_truncate_and_fallback():
    kept, removed = oracle.truncate_tail_blocks([5, 9, 2, 7], 17, 16)
    assert kept == [5, 9] and removed == [2, 7]
    assert oracle.truncate_tail_blocks([5, 9], 0, 16) == ([], [5, 9])
    assert oracle.fallback_keep_indices(10, 4, 0, False) == [6, 7, 8, 9]
    assert oracle.fallback_keep_indices(10, 4, 2, True) == [0, 1, 8, 9]
    assert oracle.fallback_keep_indices(10, 4, 5, True) is None
    assert oracle.fallback_keep_indices(3, 4, 0, False) == [0, 1, 2]


# ------------------------------------------------------------------------------------------ benchmark shapes
@pytest.fixture(scope="module")
def bench_shape_cases():
    import numpy as np
    from conftest import GOLDEN
    return np.load(GOLDEN / "bench_shape_cases.npz")


@pytest.fixture(scope="module")
def shipped_stats_cases():
    import numpy as np
    from conftest import GOLDEN
    return np.load(GOLDEN / "shipped_stats_cases.npz")


@pytest.mark.parametrize("name", ["c0_exact", "c1_slice"])
def test_checker_matches_reference_at_benchmark_shapes(manifest, bench_shape_cases, name):
    """The single-layer configuration exactly (4096 tokens, budget 2048) and a 32768-token, two-layer slice: the
    checker's keep sets and compacted caches equal the reference's own outputs."""
    p = manifest["bench_shape_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    assert tensor_sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches) == p["input_sha256"]
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    keep = oracle.select_group_per_head(layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T,
                                        p["round_start"], p["budget"], window_size=p["window"], kv_axis=p["kv_axis"])
    assert torch.equal(keep, torch.from_numpy(bench_shape_cases[f"{name}/keep"]).long())
    for l, c in enumerate(caches):
        oracle.compact_per_head(c, block_ids, bs, keep, T, kv_axis=p["kv_axis"])
        assert tensor_sha(c) == p["cache_out_sha256"][l]


def test_checker_matches_reference_on_all_layers_of_shipped_qwen3_stats(manifest, shipped_stats_cases):
    import synth
    p = manifest["shipped_stats_cases"]["cases"]["qwen3_8b_all_layers"]
    _, caches, block_ids = build_paged_case(p)
    assert tensor_sha(*caches) == p["input_sha256"]
    z = shipped_stats_cases
    stats = synth.SyntheticStats(torch.from_numpy(z["qwen3_8b_all_layers/q_mean_real"]),
                                 torch.from_numpy(z["qwen3_8b_all_layers/q_mean_imag"]),
                                 torch.from_numpy(z["qwen3_8b_all_layers/q_abs_mean"]),
                                 synth.rope_inv_freq(128, 1e6), 128, "half")
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    keep = oracle.select_group_per_head(layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T,
                                        p["round_start"], p["budget"], window_size=p["window"], kv_axis=0)
    assert torch.equal(keep, torch.from_numpy(z["qwen3_8b_all_layers/keep"]).long())
    for l, want in ((0, p["cache_out_sha256_first_last"][0]), (len(caches) - 1, p["cache_out_sha256_first_last"][1])):
        oracle.compact_per_head(caches[l], block_ids, bs, keep, T, kv_axis=0)
        assert tensor_sha(caches[l]) == want


def test_checker_matches_reference_on_gpt_oss_yarn_stats(manifest, shipped_stats_cases):
    """head_dim 64, 8 query heads per KV head, YaRN frequencies: the product's own frequency formulas reproduce the
    inv_freq the fixture was generated with, and the checker reproduces the reference's keep set."""
    import synth
    from triattention_b200 import rope
    p = manifest["shipped_stats_cases"]["cases"]["gpt_oss_yarn"]
    z = shipped_stats_cases
    inv = torch.from_numpy(z["gpt_oss_yarn/inv_freq"])
    spec = rope.rope_spec_from_parameters(64, p["theta"], p["rope_scaling"])
    assert torch.equal(spec.inv_freq, inv) and spec.attention_factor == pytest.approx(p["attention_factor"])
    stats = synth.SyntheticStats(torch.from_numpy(z["gpt_oss_yarn/q_mean_real"]), torch.from_numpy(z["gpt_oss_yarn/q_mean_imag"]),
                                 torch.from_numpy(z["gpt_oss_yarn/q_abs_mean"]), inv, 64, "half")
    from golden_cases import build_stats_case
    caches, block_ids = build_stats_case(p, inv)
    assert tensor_sha(*caches) == p["input_sha256"] and block_ids == p["block_ids"]
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    keep = oracle.select_group_per_head(layers, stats_by_layer(stats), inv, oracle.geometric_offsets(), T,
                                        p["round_start"], p["budget"], window_size=p["window"], kv_axis=0)
    assert torch.equal(keep, torch.from_numpy(z["gpt_oss_yarn/keep"]).long())
    for l, c in enumerate(caches):
        oracle.compact_per_head(c, block_ids, bs, keep, T, kv_axis=0)
        assert tensor_sha(c) == p["cache_out_sha256"][l]


def test_stats_loader_reproduces_the_reference_loader_on_shipped_files(manifest):
    """Every statistics file the reference ships, through this package's loader: metadata scalars and a hash over all
    per-layer tensors equal what the reference's own loader returned when the fixture was generated.  Needs the
    reference checkout for the files themselves (skipped where it is absent)."""
    import hashlib
    import os
    from pathlib import Path
    from conftest import REPO
    from triattention_b200 import stats as stats_mod
    ref_root = Path(os.environ.get("TRIATTN_REFERENCE_ROOT", str(REPO.parent / "reference")))
    files = manifest["stats_loader_cases"]["files"]
    if not all((ref_root / k.split("|")[0]).exists() for k in files):
        pytest.skip("statistics files of the reference checkout not present")
    for key, want in files.items():
        rel, kv = key.split("|kv=")
        nkv = None if kv == "None" else int(kv)
        if "error" in want:
            with pytest.raises(Exception):
                stats_mod.load_frequency_stats(ref_root / rel, num_kv_heads=nkv)
            continue
        md, hs = stats_mod.load_frequency_stats(ref_root / rel, num_kv_heads=nkv)
        for k, v in want["metadata"].items():
            assert md[k] == v, (key, k)
        assert float(md.get("rope_theta", 0.0)) == want["rope_theta"] and ("inv_freq" in md) == want["has_inv_freq"]
        assert sorted(int(l) for l in hs) == want["layers"]
        h = hashlib.sha256()
        for l in sorted(hs):
            for name in ("q_mean_complex", "q_abs_mean", "freq_scale_sq"):
                h.update(hs[l][name].contiguous().numpy().tobytes())
        assert h.hexdigest() == want["tensors_sha256"], key
