"""GPU parity of the Python mirror of the reference interface: selector modes, hook, batched engine, dense API."""
from __future__ import annotations

import types

import pytest
import torch

import oracle
from conftest import np_to_bf16, tensor_sha
from golden_cases import build_paged_case, stats_by_layer
from gpu_utils import device_stats, keep_sets_match_modulo_near_ties, score_tolerance_ok
from triattention_b200 import _native, engine, hook as hook_mod, kv_compaction, ops
import synth
from triattention_b200.compressor import TriAttentionCompressor, compute_scores
from triattention_b200.config import TriAttentionConfig, TriAttentionRuntimeConfig
from triattention_b200.selector import build_triattention_selector
from triattention_b200.signals import CompressionSignal

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cfg(p, stats_path, **kw):
    base = dict(
        kv_budget=p["budget"], window_size=p["window"], sparse_stats_path=stats_path,
        sparse_score_aggregation=p.get("aggregation", "mean"), sparse_normalize_scores=p.get("normalize", True),
        pruning_mode=p.get("pruning_mode", "per_head"),
        per_head_selection_semantics=p.get("semantics", "hf_aligned_global_per_head"),
        layer_perhead_aggregation=p.get("layer_perhead_aggregation", "max"),
        allow_per_layer_mode=p.get("pruning_mode", "per_head") == "per_layer",
        protect_prefill=p.get("protect_prefill", False))
    base.update(kw)
    cfg = TriAttentionRuntimeConfig(**base)
    cfg.validate()
    return cfg


def _register(caches, p):
    for c in caches:
        if int(c.shape[0]) == 2 and int(c.shape[1]) == 2:
            kv_compaction.register_kv_layout_axis_hint(c, p["kv_axis"])


@pytest.mark.parametrize("name", ["tiny_group", "chunked_group", "c0_like", "llama3_nonorm", "max_agg_prefill", "d64_g8"])
def test_group_selector_matches_reference_keep(manifest, selector_cases, tmp_path, name):
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    _, sel_group, status = build_triattention_selector(_cfg(p, sp))
    assert status == "enabled" and sel_group._supports_paged_group
    dc = [c.to(DEV) for c in caches]
    _register(dc, p)
    T, bs = p["total_tokens"], p["block_size"]

    def _iter():
        for l, c in enumerate(dc):
            yield l, c, block_ids, bs

    res = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, total_tokens=T,
                    prefill_len=p.get("prefill_len", 0), protect_prefill=p.get("protect_prefill", False),
                    round_start=p["round_start"], budget_total=min(p["budget"], T))
    assert res["mode"] == "per_head" and res["semantic"] == "hf_aligned_global_per_head"
    assert res["indices"].dtype == torch.int64 and res["debug_recent_count"] == min(p["window"], T)
    ref_keep = torch.from_numpy(selector_cases[f"{name}/keep"]).long()
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    ref_final = oracle.final_scores_group_per_head(
        layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"],
        window_size=p["window"], prefill_len=p.get("prefill_len", 0), protect_prefill=p.get("protect_prefill", False),
        normalize=p.get("normalize", True), aggregation=p.get("aggregation", "mean"), kv_axis=p["kv_axis"])
    ok, nd = keep_sets_match_modulo_near_ties(res["indices"].cpu(), ref_keep, ref_final)
    assert ok, nd
    # under budget: identity
    ident = sel_group(layer_inputs=None, layer_input_iter=None, layer_kv_iter=_iter, total_tokens=T, prefill_len=0,
                      protect_prefill=False, round_start=T, budget_total=T)
    assert torch.equal(ident["indices"].cpu(), torch.arange(T).expand(p["num_kv_heads"], -1))


@pytest.mark.parametrize("name,mode", [("legacy_layer_local", "per_head"), ("per_layer_shared", "shared"),
                                       ("plph_mean", "per_head")])
def test_layer_local_selector_modes(manifest, selector_cases, tmp_path, name, mode):
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    sel_layer, sel_group, _ = build_triattention_selector(_cfg(p, sp))
    T, bs = p["total_tokens"], p["block_size"]
    sl = stats_by_layer(stats)
    for l, c in enumerate(caches):
        dcache = c.to(DEV)
        res = sel_layer(keys_dense=None, kv_cache=dcache, block_ids=torch.as_tensor(block_ids), block_size=bs,
                        total_tokens=T, prefill_len=0, protect_prefill=False, layer_idx=l,
                        round_start=p["round_start"], budget_total=p["budget"])
        assert res["mode"] == mode
        ref_keep = torch.from_numpy(selector_cases[f"{name}/keep_l{l}"]).long()
        got = res["indices"].cpu()
        # any index that differs from the reference's keep set must be a near-tie at the cut-off (1e-3 sigma_row)
        _, ref_rows = oracle.select_layer_local(
            c, block_ids, bs, sl[l], stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"], p["budget"],
            mode=mode, group_agg="mean" if name == "plph_mean" else "max", reduce_stats=name != "plph_mean",
            window_size=p["window"], kv_axis=p["kv_axis"], return_scores=True)
        ok, nd = keep_sets_match_modulo_near_ties(got.view(ref_rows.shape[0], -1), ref_keep.view(ref_rows.shape[0], -1),
                                                  ref_rows)
        assert ok, (l, nd)
        # compaction through the mirrored API, whole region equal to the checker with the same keep set
        exp = c.clone()
        if mode == "shared":
            n = kv_compaction.compact_request_kv_in_place(dcache, block_ids, bs, res["indices"], T)
            oracle.compact_shared(exp, block_ids, bs, got, T, preserve_dropped_tokens=True, kv_axis=0)
        else:
            n = kv_compaction.compact_request_kv_in_place_per_head(dcache, block_ids, bs, res["indices"], T)
            oracle.compact_per_head(exp, block_ids, bs, got, T, preserve_dropped_tokens=True, kv_axis=0)
        assert n == p["budget"]
        assert torch.equal(dcache.cpu().view(torch.int16), exp.view(torch.int16))


def test_compaction_api_errors():
    g = torch.Generator().manual_seed(3)
    cache = torch.randn((2, 8, 16, 2, 128), generator=g).to(torch.bfloat16).to(DEV)
    ids = [3, 1, 5, 2]
    with pytest.raises(IndexError):
        kv_compaction.compact_request_kv_in_place_per_head(cache, ids, 16, torch.tensor([[0, 70], [1, 2]]), 64)
    with pytest.raises(ValueError, match="duplicates"):
        kv_compaction.compact_request_kv_in_place_per_head(cache, ids, 16, torch.tensor([[1, 1], [1, 2]]), 64)
    with pytest.raises(ValueError, match="head count"):
        kv_compaction.compact_request_kv_in_place_per_head(cache, ids, 16, torch.tensor([[1, 2]]), 64)
    with pytest.raises(ValueError, match="2D"):
        kv_compaction.compact_request_kv_in_place_per_head(cache, ids, 16, torch.tensor([1, 2]), 64)
    with pytest.raises(IndexError):
        kv_compaction.compact_request_kv_in_place(cache, ids, 16, [0, 5, 64], 64)
    with pytest.raises(ValueError, match="duplicates"):
        kv_compaction.compact_request_kv_in_place(cache, ids, 16, [0, 5, 5], 64)
    with pytest.raises(IndexError):
        kv_compaction.compact_request_kv_in_place(cache, ids, 16, [0, 5, 9], 100)   # needs 7 blocks, 4 given
    assert kv_compaction.compact_request_kv_in_place(cache, ids, 16, [], 64) == 0
    before = cache.clone()
    assert kv_compaction.compact_request_kv_in_place(cache, ids, 16, list(range(10)), 64) == 10   # identity
    assert torch.equal(cache, before)
    amb = torch.zeros((2, 2, 16, 2, 128), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="Ambiguous"):
        kv_compaction.compact_request_kv_in_place(amb, [0, 1], 16, [1, 2], 20)


def test_hook_on_gpu_matches_reference_results(manifest, tmp_path):
    hc = manifest["hook_cases"]
    p, want = hc["params"], hc["results"]
    stats, caches, block_ids = build_paged_case(p)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    T = p["total_tokens"]
    for preserve in (True, False):
        dc = [c.to(DEV) for c in caches]
        cfg = TriAttentionRuntimeConfig(kv_budget=p["budget"], window_size=p["window"], sparse_stats_path=sp,
                                        preserve_dropped_tokens=preserve)
        runner = types.SimpleNamespace(
            requests={"r0": types.SimpleNamespace(block_ids=(list(block_ids),), num_computed_tokens=T),
                      "r1": types.SimpleNamespace(block_ids=(list(block_ids[:8]),), num_computed_tokens=100)},
            kv_caches=dc, cache_config=types.SimpleNamespace(block_size=p["block_size"]))
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
        assert hook(req_id="r0", signal=sig("r0", T + 1), scheduler_output=so) == want["compacted"]
        assert [list(g) for g in runner.requests["r0"].block_ids] == want["block_ids_after"]
        if preserve:
            # same keep set as the reference (no near-tie at the cut-off in this fixture): byte-identical caches
            assert [tensor_sha(c) for c in dc] == p["cache_out_sha256"]
        runner.requests["r0"].num_computed_tokens = T + 40
        assert hook(req_id="r0", signal=sig("r0", 256 + 40 + 1), scheduler_output=so) == want["deferred"]


def test_batched_engine_equals_per_request_calls():
    """Ragged batch (different lengths, round starts, budgets) in one native call == one call per request."""
    gen = torch.Generator().manual_seed(21)
    L, Hq, Hkv, D, bs = 3, 8, 2, 128, 16
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    lens, budgets, starts = [700, 37, 2500, 1024], [256, 64, 512, 1024], [700, 5000, 2500, 70000]
    nblk = [(t + bs - 1) // bs for t in lens]
    perm = synth.random_block_ids(sum(nblk), sum(nblk) + 9, gen)
    ids, o = [], 0
    for n in nblk:
        ids.append(perm[o:o + n])
        o += n
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(sum(nblk) + 9, bs, Hkv, D, kv_axis=1)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 1, ids[b], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    dstats = device_stats(stats, oracle.geometric_offsets())
    batched = [c.to(DEV) for c in caches]
    comp = engine.PagedCompressor(dstats, window=32)
    res = comp.compress(ops.PagedCacheView.from_layers(batched, kv_axis=1), ids, lens, starts, budgets)
    assert res.device_status == 0 and res.keep_counts == [256, 37, 512, 1024]
    single = [c.to(DEV) for c in caches]
    view1 = ops.PagedCacheView.from_layers(single, kv_axis=1)
    for b in range(len(lens)):
        r1 = engine.PagedCompressor(dstats, window=32).compress(view1, [ids[b]], [lens[b]], [starts[b]], [budgets[b]])
        k = r1.keep_counts[0]
        assert torch.equal(r1.keep[0, :, :k], res.keep[b, :, :k])
        assert r1.kept_block_ids[0] == res.kept_block_ids[b] == ids[b][: (k + bs - 1) // bs]
        assert r1.removed_block_ids[0] == res.removed_block_ids[b]
    for a, c in zip(batched, single):
        assert torch.equal(a, c)
    # the request that fits its budget is untouched and keeps the identity set
    assert torch.equal(res.keep[1, :, :37].cpu(), torch.arange(37, dtype=torch.int32).expand(Hkv, -1))
    with pytest.raises(IndexError):
        comp.compress(ops.PagedCacheView.from_layers(batched, kv_axis=1), [ids[0][:3]], [700], [700], [256])


def test_dense_api(manifest, score_cases, tmp_path):
    a = score_cases
    v = manifest["score_cases"]["variants"][0]
    keys = np_to_bf16(a["keys_0"]).to(DEV)
    cfg = TriAttentionConfig(score_aggregation=v["aggregation"], rope_style=v["rope_style"])
    hs = {"q_mean_complex": torch.stack([torch.from_numpy(a["q_mean_real"]), torch.from_numpy(a["q_mean_imag"])], -1).to(DEV),
          "q_abs_mean": torch.from_numpy(a["q_abs_mean"]).to(DEV)}
    got = compute_scores(keys, None, hs, torch.from_numpy(a["omega"]).to(DEV), torch.from_numpy(a["offsets"]).to(DEV),
                         torch.from_numpy(a["freq_scale_sq"]).to(DEV), cfg, round_start=v["round_start"])
    ok, worst = score_tolerance_ok(got.cpu(), torch.from_numpy(a["scores_0"]))
    assert ok, worst
    with pytest.raises(_native.NativeLibraryError):
        compute_scores(keys.cpu(), None, hs, None, None, None, cfg, round_start=1)

    # dense compress(): budget tokens per head, window kept, gathered K/V consistent with the indices
    gen = torch.Generator().manual_seed(5)
    H, T, D = 4, 600, 128
    inv = synth.rope_inv_freq(D, 1e6)
    st = synth.make_stats(1, H, D, inv, gen)
    sp = tmp_path / "d.pt"
    synth.save_stats_pt(st, sp)
    comp = TriAttentionCompressor(TriAttentionConfig(kv_budget=128, divide_length=64, window_size=16, stats_path=sp,
                                                     device=torch.device(DEV)))
    k = synth.make_rotated_keys(H, T, D, inv, gen).permute(1, 0, 2).unsqueeze(0).to(DEV)
    vv = synth.make_values(H, T, D, gen).permute(1, 0, 2).unsqueeze(0).to(DEV)
    ck, cv, idx = comp.compress(k, vv, layer_idx=0)
    assert ck.shape == (1, H, 128, D) and idx.shape == (1, H, 128)
    assert bool((idx[0, :, -16:] == torch.arange(T - 16, T, device=DEV)).all())
    assert torch.equal(ck[0, 2], k[0, 2, idx[0, 2]]) and torch.equal(cv[0, 1], vv[0, 1, idx[0, 1]])
    raw = oracle.score_keys_reference(k.cpu(), st.q_mean_real[0], st.q_mean_imag[0], st.q_abs_mean[0],
                                      torch.ones(H, D // 2), inv, oracle.geometric_offsets(), T)[0]
    mean, std = oracle.streaming_moments(raw, chunk_tokens=T)
    z = (raw - mean[:, None]) / std[:, None]
    z[:, -16:] = float("inf")
    ok, nd = keep_sets_match_modulo_near_ties(idx[0].cpu(), oracle.topk_lowest_index(z, 128), z)
    assert ok, nd
    small_k, _, small_idx = comp.compress(k[:, :, :100], vv[:, :, :100])
    assert small_k.shape[2] == 100 and torch.equal(small_idx.cpu(), torch.arange(100))


@pytest.mark.parametrize("agg", ["mean", "max"])
def test_engine_cuda_graph_replay_matches_eager(agg):
    """The batched step replayed from a CUDA graph gives the keep sets and caches of the eager call (with max
    aggregation the capture also holds the kernel that stamps the tensor-core scorer's tensor maps)."""
    from gpu_utils import device_stats
    from triattention_b200 import _native, engine

    offset_agg = _native.OFFSETS_MAX if agg == "max" else _native.OFFSETS_MEAN

    gen = torch.Generator().manual_seed(synth.seed_for(3, 5))
    L, Hq, Hkv, D, bs, lens, budget = 2, 8, 2, 128, 16, [300, 257], 128
    inv = synth.rope_inv_freq(D, 5e5)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    nblk = [(t + bs - 1) // bs for t in lens]
    total = sum(nblk) + 3
    perm = synth.random_block_ids(sum(nblk), total, gen)
    ids = [perm[:nblk[0]], perm[nblk[0]:]]
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(total, bs, Hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    dstats = device_stats(stats, oracle.geometric_offsets())
    eager = engine.PagedCompressor(dstats, window=32, offset_agg=offset_agg)
    dc = [c.cuda() for c in caches]
    ref = eager.compress(ops.PagedCacheView.from_layers(dc, kv_axis=0), ids, lens, lens, [budget] * 2)
    ref_keep, ref_caches = ref.keep.clone(), [c.clone() for c in dc]

    graphed = engine.PagedCompressor(dstats, window=32, use_cuda_graph=True, offset_agg=offset_agg)
    work = [c.cuda() for c in caches]
    view = ops.PagedCacheView.from_layers(work, kv_axis=0)
    for round_ in range(4):  # eager, capture + replay, replay, replay
        for w, c in zip(work, caches):
            w.copy_(c)
        res = graphed.compress(view, ids, lens, lens, [budget] * 2)
        assert res.device_status == 0
        assert torch.equal(res.keep, ref_keep), f"round {round_}"
        for w, r in zip(work, ref_caches):
            assert torch.equal(w.view(torch.int16), r.view(torch.int16)), f"round {round_}"
    assert len(graphed._graphs) == 1


def test_flat_pool_entry_matches_slot_arithmetic():
    """The SGLang-shaped entry (token-granular pool, req_to_token table) against plain advanced indexing on the CPU,
    i.e. the gather / scatter the reference performs (sglang/kv_compaction.py:372-402)."""
    from triattention_b200 import flat_pool
    gen = torch.Generator().manual_seed(77)
    L, H, D, pool, T, budget = 3, 4, 128, 700, 400, 150
    kb = [torch.randn((pool, H, D), generator=gen).to(torch.bfloat16) for _ in range(L)]
    vb = [torch.randn((pool, H, D), generator=gen).to(torch.bfloat16) for _ in range(L)]
    req_to_token = torch.zeros((3, 512), dtype=torch.int32)
    slots = torch.randperm(pool - 1, generator=gen)[:T] + 1
    req_to_token[1, :T] = slots.int()
    keep = torch.stack([torch.sort(torch.randperm(T, generator=gen)[:budget]).values for _ in range(H)])
    dk, dv = [x.to(DEV) for x in kb], [x.to(DEV) for x in vb]
    n = flat_pool.compact_request_kv_in_place_per_head(dk, dv, req_to_token.to(DEV), 1, keep.to(DEV), T, target_layers=[0, 2])
    assert n == budget
    head = torch.arange(H).unsqueeze(1).expand(-1, budget)
    src, dst = slots[keep], slots[:budget].unsqueeze(0).expand(H, -1)
    for l in range(L):
        ek, ev = kb[l].clone(), vb[l].clone()
        if l != 1:
            gk, gv = ek[src, head].clone(), ev[src, head].clone()
            ek[dst, head], ev[dst, head] = gk, gv
        assert torch.equal(dk[l].cpu().view(torch.int16), ek.view(torch.int16)), l
        assert torch.equal(dv[l].cpu().view(torch.int16), ev.view(torch.int16)), l
    with pytest.raises(IndexError):
        flat_pool.compact_request_kv_in_place_per_head(dk, dv, req_to_token.to(DEV), 1, (keep + 300).to(DEV), T)
    with pytest.raises(ValueError, match="sorted ascending"):
        flat_pool.compact_request_kv_in_place_per_head(dk, dv, req_to_token.to(DEV), 1, keep.flip(1).to(DEV), T)
    with pytest.raises(ValueError, match="exceeds effective_len"):
        flat_pool.compact_request_kv_in_place_per_head(dk, dv, req_to_token.to(DEV), 1, keep.to(DEV), 100)


def test_layer_shared_step_with_a_single_local_kv_head():
    """A rank that holds one KV head has nothing to reduce over heads: the layer-shared step then finalises with the
    per-head kernel.  Its keep rows must equal the ones the head-reducing kernel gives on the same cache."""
    from gpu_utils import block_table_tensor, device_stats
    from triattention_b200 import _native, engine

    gen = torch.Generator().manual_seed(synth.seed_for(3, 9))
    L, Hq, Hkv, D, bs, lens, budgets = 3, 4, 1, 128, 16, [700, 333], [256, 128]
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    nblk = [(t + bs - 1) // bs for t in lens]
    perm = synth.random_block_ids(sum(nblk), sum(nblk) + 4, gen)
    ids = [perm[:nblk[0]], perm[nblk[0]:]]
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(sum(nblk) + 4, bs, Hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    ds = device_stats(stats, oracle.geometric_offsets())
    work = [c.cuda() for c in caches]
    view = ops.PagedCacheView.from_layers(work, kv_axis=0)
    res = engine.compress_layer_shared(view, ds, ids, lens, lens, budgets, window=32, process_group=False,
                                       reduce_stats_to_kv_heads=False)
    assert res.device_status == 0
    # the same selection through the staged entry points with the head reduction spelled out
    ref_caches = [c.cuda() for c in caches]
    rview = ops.PagedCacheView.from_layers(ref_caches, kv_axis=0)
    bt = block_table_tensor(ids)
    layout = rview.layout(2, Hq // Hkv, bt.shape[1])
    meta = torch.tensor([lens, lens, budgets], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    w = ops.prep_weights_fused(ds, meta[1])
    raw, mom = ops.score_paged(rview, layout, bt, meta[0], w, status=status)
    fin = ops.finalize_scores(layout, raw, mom, meta[0], None, 32, True, _native.REDUCE_MAX, _native.REDUCE_MAX,
                              _native.REDUCE_NONE)
    keep = ops.select_topk(fin.view(L * 2, fin.shape[-1]), meta[0], meta[2], 2, 1, max(budgets), status)
    assert int(status.item()) == 0
    assert torch.equal(res.keep.view(L * 2, -1), keep)


def test_batched_hook_equals_the_per_request_hook(tmp_path):
    """All triggered requests of a step through ``triattention_apply_compression_batch`` (one native call) against
    the per-request hook called request after request: same result dictionaries, block tables and cache bytes."""
    gen = torch.Generator().manual_seed(synth.seed_for(5, 1))
    L, Hq, Hkv, D, bs, budget, window = 2, 8, 2, 128, 16, 256, 32
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    lens = {"a": 900, "b": 100, "c": 640, "d": 1301}       # b is under budget, the others compress
    nblk = {r: (t + bs - 1) // bs for r, t in lens.items()}
    perm = synth.random_block_ids(sum(nblk.values()), sum(nblk.values()) + 6, gen)
    ids, o = {}, 0
    for r, n in nblk.items():
        ids[r] = perm[o:o + n]
        o += n
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(sum(nblk.values()) + 6, bs, Hkv, D, kv_axis=0)
        for r, t in lens.items():
            synth.write_tokens_to_paged(c, 0, ids[r], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)

    def make():
        dc = [c.to(DEV) for c in caches]
        cfg = TriAttentionRuntimeConfig(kv_budget=budget, window_size=window, sparse_stats_path=sp)
        runner = types.SimpleNamespace(
            requests={r: types.SimpleNamespace(block_ids=(list(ids[r]),), num_computed_tokens=t) for r, t in lens.items()},
            kv_caches=dc, cache_config=types.SimpleNamespace(block_size=bs))
        hook_mod.install_runner_compression_hook(runner, cfg)
        return runner, dc

    def sig(req):
        return CompressionSignal(req_id=req, should_compress=True, reason="length_threshold",
                                 estimated_cache_len=lens[req] + 1, step=3, kv_usage=None, protect_prefill=False,
                                 prefill_len=0, scheduled_tokens=1)

    so = types.SimpleNamespace(num_scheduled_tokens={r: 1 for r in lens})
    order = ["a", "b", "zz", "c", "d"]                      # zz does not exist
    one, one_caches = make()
    want = {r: one.triattention_apply_compression(req_id=r, signal=sig(r) if r in lens else
                                                  CompressionSignal(req_id=r, should_compress=True, reason="x",
                                                                    estimated_cache_len=5, step=3, kv_usage=None,
                                                                    protect_prefill=False, prefill_len=0, scheduled_tokens=1),
                                                  scheduler_output=so) for r in order}
    many, many_caches = make()
    reqs = [(r, sig(r) if r in lens else CompressionSignal(req_id=r, should_compress=True, reason="x", estimated_cache_len=5,
                                                            step=3, kv_usage=None, protect_prefill=False, prefill_len=0,
                                                            scheduled_tokens=1)) for r in order]
    got = many.triattention_apply_compression_batch(reqs, so)
    assert got == want
    assert want["a"]["applied"] and want["c"]["applied"] and want["d"]["applied"] and not want["b"]["applied"]
    for r in lens:
        assert many.requests[r].block_ids == one.requests[r].block_ids
    for a, b in zip(many_caches, one_caches):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # a second round on the same runners: the compressed requests are now under budget + slack on both paths
    assert many.triattention_apply_compression_batch(reqs, so) == {
        r: one.triattention_apply_compression(req_id=r, signal=s, scheduler_output=so) for r, s in reqs}


def test_runner_proxy_step_with_the_real_hook(tmp_path):
    """A whole worker step through ``worker_runner.TriAttentionModelRunner`` with the installed hook: the triggered
    requests of the step are compacted in one native call, the events reach the engine's output, the request-state
    store and the block lists are updated, and the caches equal those of the per-request hook."""
    from triattention_b200 import worker_runner

    gen = torch.Generator().manual_seed(synth.seed_for(5, 2))
    L, Hq, Hkv, D, bs, budget, window = 2, 8, 2, 128, 16, 256, 32
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    sp = tmp_path / "s.pt"
    synth.save_stats_pt(stats, sp)
    lens = {"a": 900, "b": 100, "c": 640}                   # b stays under the budget
    nblk = {r: (t + bs - 1) // bs for r, t in lens.items()}
    perm = synth.random_block_ids(sum(nblk.values()), sum(nblk.values()) + 6, gen)
    ids, o = {}, 0
    for r, n in nblk.items():
        ids[r] = perm[o:o + n]
        o += n
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(sum(nblk.values()) + 6, bs, Hkv, D, kv_axis=0)
        for r, t in lens.items():
            synth.write_tokens_to_paged(c, 0, ids[r], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    cfg = TriAttentionRuntimeConfig(kv_budget=budget, divide_length=64, window_size=window, sparse_stats_path=sp,
                                    log_decisions=False)

    def make():
        dc = [c.to(DEV) for c in caches]
        runner = types.SimpleNamespace(
            requests={r: types.SimpleNamespace(block_ids=(list(ids[r]),), num_computed_tokens=t) for r, t in lens.items()},
            kv_caches=dc, cache_config=types.SimpleNamespace(block_size=bs))
        runner.execute_model = lambda scheduler_output, intermediate_tensors=None: types.SimpleNamespace(tag="out")
        hook_mod.install_runner_compression_hook(runner, cfg)
        return runner, dc

    def sig(req, should=True):
        return CompressionSignal(req_id=req, should_compress=should, reason="length_threshold" if should else "none",
                                 estimated_cache_len=lens[req] + 1, step=2, kv_usage=None, protect_prefill=False,
                                 prefill_len=lens[req], scheduled_tokens=1)

    def step_output(step, signals):
        return types.SimpleNamespace(triattention_step=step, triattention_signals=signals,
                                     num_scheduled_tokens={r: 1 for r in lens}, scheduled_new_reqs=[],
                                     finished_req_ids=[])

    # reference run: the per-request hook, request after request, on its own copy of the caches
    one, one_caches = make()
    so = step_output(2, {})
    want = {r: one.triattention_apply_compression(req_id=r, signal=sig(r), scheduler_output=so) for r in lens}

    runner, dc = make()
    proxy = worker_runner.TriAttentionModelRunner(runner, cfg)
    out = proxy.execute_model(step_output(2, {r: sig(r) for r in lens}))
    events = out.triattention_compression_events
    assert [(e["req_id"], e["status"]) for e in events] == [("a", "applied"), ("b", "skipped"), ("c", "applied")]
    for e in events:
        assert e["reason"] == want[e["req_id"]]["reason"]
        if e["status"] == "applied":
            assert e["cache_len_after"] == budget and e["block_reclaim"]["groups"][0]["block_ids_after"] == \
                list(ids[e["req_id"]][: budget // bs])
    for r in lens:
        assert runner.requests[r].block_ids == one.requests[r].block_ids
    for x, y in zip(dc, one_caches):
        assert torch.equal(x.view(torch.int16), y.view(torch.int16))
    states = proxy.snapshot_states()
    assert states["a"].compression_count == 1 and states["c"].compression_count == 1 and states["b"].compression_count == 0
    assert states["a"].current_cache_len == budget + 1
    # next step: nothing from the scheduler, and the worker's own count (257 + 1) is below budget + slack: no trigger
    snap = [c.clone() for c in dc]
    out = proxy.execute_model(step_output(3, {}))
    assert out.triattention_compression_events == []
    assert all(torch.equal(x, y) for x, y in zip(dc, snap))
