"""GPU checks of the fused step's plumbing: one-launch weight prep, layer-chunked workspaces, the length clamp
of the top-k, the wait-timeout status path, and full parity against the CPU checker at the benchmark length."""
from __future__ import annotations

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

import oracle
import synth
from gpu_utils import (block_table_tensor, device_stats, keep_sets_match_modulo_near_ties, raw_to_reference_layout,
                       score_tolerance_ok)
from triattention_b200 import _native, build, engine, ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
BS = 16
REPO = Path(__file__).resolve().parent.parent


def _stats_dict(stats):
    return {l: {"q_mean_real": stats.q_mean_real[l], "q_mean_imag": stats.q_mean_imag[l],
                "q_abs_mean": stats.q_abs_mean[l], "freq_scale_sq": torch.ones_like(stats.q_abs_mean[l])}
            for l in range(stats.num_layers)}


def _build_case(L, Hq, Hkv, D, lens, seed, theta=1e6):
    gen = torch.Generator().manual_seed(seed)
    inv = synth.rope_inv_freq(D, theta)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    nblk = [(t + BS - 1) // BS for t in lens]
    total = sum(nblk) + 7
    perm = synth.random_block_ids(sum(nblk), total, gen)
    ids, o = [], 0
    for n in nblk:
        ids.append(perm[o:o + n])
        o += n
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(total, BS, Hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], BS, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    return stats, caches, ids, inv


@pytest.mark.parametrize("agg", [_native.OFFSETS_MEAN, _native.OFFSETS_MAX])
@pytest.mark.parametrize("flags", [0, _native.FLAG_DISABLE_MLR, _native.FLAG_DISABLE_TRIG])
def test_fused_prep_is_bit_identical_and_clears_moments(agg, flags):
    gen = torch.Generator().manual_seed(91)
    L, Hq, D, B = 5, 12, 128, 7
    stats = synth.make_stats(L, Hq, D, synth.rope_inv_freq(D, 1e6), gen)
    ds = device_stats(stats, oracle.geometric_offsets())
    rs = torch.tensor([4096, 1, 33000, 131071, 2176, 70000, 12345], dtype=torch.int32, device=DEV)
    want = ops.prep_weights(ds, rs, agg, flags)
    mom = torch.full((L, B, Hq, 2), 3.5, dtype=torch.float64, device=DEV)
    got = ops.prep_weights_fused(ds, rs, agg, flags, moments_to_clear=mom)
    torch.cuda.synchronize()
    assert got.shape == want.shape and torch.equal(got.view(torch.int32), want.view(torch.int32))
    assert int(torch.count_nonzero(mom)) == 0
    # a single request and a single (layer, head) row
    one = ops.DeviceStats(ds.q_mean_real[:1, :1].contiguous(), ds.q_mean_imag[:1, :1].contiguous(),
                          ds.q_abs_mean[:1, :1].contiguous(), ds.freq_scale_sq[:1, :1].contiguous(), ds.omega, ds.offsets)
    assert torch.equal(ops.prep_weights_fused(one, rs[:1], agg, flags), ops.prep_weights(one, rs[:1], agg, flags))


@pytest.mark.parametrize("g,hkv", [(4, 2), (8, 1)])
def test_layer_chunked_workspace_gives_identical_results(g, hkv):
    """A workspace that holds the raw scores of one, two or all layers: same keep sets, same caches, bit for bit."""
    L, D, lens, budget, window = 5, 128, [1500, 700, 2048], [512, 300, 512], 64
    stats, caches, ids, inv = _build_case(L, hkv * g, hkv, D, lens, seed=1717)
    ds = device_stats(stats, oracle.geometric_offsets())
    results = []
    full_ws = None
    for cap in (None, 0, "two"):
        dc = [c.to(DEV) for c in caches]
        view = ops.PagedCacheView.from_layers(dc, kv_axis=0)
        comp = engine.PagedCompressor(ds, window=window)
        if cap is not None:
            layout = view.layout(len(lens), g, max((t + BS - 1) // BS for t in lens))
            lo = ops.compress_workspace_bytes_min(layout, 17, _native.OFFSETS_MEAN, max(budget))
            hi = ops.compress_workspace_bytes(layout, 17, _native.OFFSETS_MEAN, max(budget))
            per_layer = (hi - lo) // (L - 1)
            comp.max_workspace_bytes = lo if cap == 0 else lo + per_layer
            full_ws = hi
        res = comp.compress(view, ids, lens, [t + 3 for t in lens], budget)
        assert res.device_status == 0
        if cap is not None:
            assert comp._workspace.numel() < full_ws
        results.append((res.keep.clone(), [c.clone() for c in dc]))
    for keep, dc in results[1:]:
        assert torch.equal(keep, results[0][0])
        assert all(torch.equal(a, b) for a, b in zip(dc, results[0][1]))
    # and the full-workspace run agrees with the checker
    layers = [(l, c, ids[0], BS) for l, c in enumerate(caches)]
    fin = oracle.final_scores_group_per_head(layers, _stats_dict(stats), inv, oracle.geometric_offsets(), lens[0],
                                             lens[0] + 3, window_size=window, kv_axis=0)
    ok, nd = keep_sets_match_modulo_near_ties(results[0][0][0, :, :budget[0]].cpu().long(),
                                              oracle.topk_lowest_index(fin, budget[0]), fin)
    assert ok, nd
    # a workspace below the minimum is refused
    dc = [c.to(DEV) for c in caches]
    view = ops.PagedCacheView.from_layers(dc, kv_axis=0)
    layout = view.layout(1, g, (lens[0] + BS - 1) // BS)
    small = torch.empty(ops.compress_workspace_bytes_min(layout, 17, 0, 64) - 256, dtype=torch.uint8, device=DEV)
    meta = torch.tensor([lens[0], lens[0], 64], dtype=torch.int32, device=DEV)
    with pytest.raises(_native.NativeLibraryError, match="workspace too small"):
        ops.compress_paged(view, layout, ds, block_table_tensor([ids[0]]), meta[0:1], meta[1:2], None, meta[2:3], 64,
                           window, workspace=small)


def test_select_clamps_a_length_beyond_the_row():
    """seq_len larger than the score row: clamped, reported in the status word, nothing read past the row."""
    rows, stride, k = 3, 200, 16
    scores = torch.randn((rows, stride), device=DEV)
    seq = torch.tensor([stride + 37], dtype=torch.int32, device=DEV)
    kc = torch.tensor([k], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    keep = ops.select_topk(scores, seq, kc, 1, rows, k, status)
    torch.cuda.synchronize()
    assert int(status.item()) & _native.DEV_BAD_LENGTH
    assert int(keep.min()) >= 0 and int(keep.max()) < stride
    want = torch.topk(scores, k, dim=1).indices.sort(dim=1).values.int()
    assert torch.equal(keep, want)


def test_wait_timeout_reports_status_and_returns():
    """The test-only library build gives every bounded wait a ~1 ms limit and lets every barrier expect 16 bytes that
    never arrive: each wait runs out after the real copies have landed, the kernels set TRIATTN_DEV_WAIT_TIMEOUT,
    drain and return; the process ends normally and the GPU stays usable (the next test runs on it)."""
    lib = build.build_library(short_wait=True)
    code = textwrap.dedent("""
        import sys, torch
        sys.path.insert(0, %r); sys.path.insert(0, %r)
        import synth
        from triattention_b200 import _native, engine, ops
        gen = torch.Generator().manual_seed(5)
        bits = []
        for hkv, g, agg in ((8, 4, 0), (2, 4, 0), (2, 4, 1)):
            L, D, T, bs = 2, 128, 700, 16
            inv = synth.rope_inv_freq(D, 1e6)
            st = synth.make_stats(L, hkv * g, D, inv, gen)
            nblk = (T + bs - 1) // bs
            ids = synth.random_block_ids(nblk, nblk + 3, gen)
            caches = []
            for _ in range(L):
                c = synth.make_paged_layer(nblk + 3, bs, hkv, D, kv_axis=0)
                synth.write_tokens_to_paged(c, 0, ids, bs, synth.make_rotated_keys(hkv, T, D, inv, gen),
                                            synth.make_values(hkv, T, D, gen))
                caches.append(c.cuda())
            off = torch.tensor([float(2 ** i) for i in range(17)])
            ds = ops.DeviceStats(st.q_mean_real.cuda(), st.q_mean_imag.cuda(), st.q_abs_mean.cuda(),
                                 torch.ones_like(st.q_abs_mean).cuda(), inv.cuda(), off.cuda())
            comp = engine.PagedCompressor(ds, window=16, offset_agg=agg)
            res = comp.compress(ops.PagedCacheView.from_layers(caches, kv_axis=0), [ids], [T], [T], [128])
            torch.cuda.synchronize()
            bits.append(res.device_status)
        x = torch.arange(10, device="cuda").sum().item()      # the context still works
        print("STATUS", *bits, x)
    """) % (str(REPO), str(REPO / "tests"))
    env = dict(os.environ, TRIATTN_B200_LIB=str(lib))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("STATUS")][-1].split()
    assert all(int(b) & _native.DEV_WAIT_TIMEOUT for b in line[1:4]), line
    assert int(line[4]) == 45
    # this process (the regular library) is unaffected
    assert torch.arange(4, device=DEV).sum().item() == 6


@pytest.mark.parametrize("hkv,g", [(8, 4), (8, 8), (1, 8)])
def test_benchmark_length_full_parity(hkv, g):
    """T = 32768, budget 2048, window 128, one request x two layers (the slice the CPU leg of the bench times):
    raw and final scores within 1e-3, keep sets equal except near-ties, compacted prefix bit-exact."""
    L, D, T, budget, window = 2, 128, 32768, 2048, 128
    stats, caches, ids, inv = _build_case(L, hkv * g, hkv, D, [T], seed=synth.seed_for(1, 5, hkv * 10 + g))
    layers = [(l, c, ids[0], BS) for l, c in enumerate(caches)]
    ref_final, ref_raws = oracle.final_scores_group_per_head(layers, _stats_dict(stats), inv, oracle.geometric_offsets(),
                                                             T, T, window_size=window, kv_axis=0, return_raw=True)
    ref_keep = oracle.topk_lowest_index(ref_final, budget)
    dc = [c.to(DEV) for c in caches]
    view = ops.PagedCacheView.from_layers(dc, kv_axis=0)
    ds = device_stats(stats, oracle.geometric_offsets())
    bt = block_table_tensor([ids[0]])
    layout = view.layout(1, g, bt.shape[1])
    meta = torch.tensor([T, T, budget, 0], dtype=torch.int32, device=DEV)
    seq, rs, kc, status = meta[0:1], meta[1:2], meta[2:3], meta[3:4]
    w = ops.prep_weights_fused(ds, rs)
    raw, mom = ops.score_paged(view, layout, bt, seq, w, status=status)
    fin = ops.finalize_scores(layout, raw, mom, seq, None, window)
    ok, worst = score_tolerance_ok(raw_to_reference_layout(raw, g, T)[:, 0].cpu(), torch.stack(ref_raws))
    assert ok, f"raw score error {worst}"
    got_fin = fin[0, 0, :, :T].cpu()
    finite = torch.isfinite(ref_final)
    assert torch.equal(torch.isfinite(got_fin), finite)
    ok, worst = score_tolerance_ok(torch.where(finite, got_fin, 0.0), torch.where(finite, ref_final, 0.0))
    assert ok, f"final score error {worst}"
    # the fused step: keep sets and compaction
    comp = engine.PagedCompressor(ds, window=window)
    res = comp.compress(view, ids, [T], [T], [budget])
    assert res.device_status == 0 and int(status.item()) == 0
    keep = res.keep[0].cpu().long()
    ok, nd = keep_sets_match_modulo_near_ties(keep, ref_keep, ref_final)
    assert ok, nd
    for l, c in enumerate(caches):
        exp = c.clone()
        oracle.compact_per_head(exp, ids[0], BS, keep, T, preserve_dropped_tokens=False, kv_axis=0)
        assert torch.equal(dc[l].cpu().view(torch.int16), exp.view(torch.int16)), l
    assert res.kept_block_ids[0] == ids[0][: budget // BS]


# ------------------------------------------------------------------------------------------ reference-generated fixtures
def _device_keep_vs_reference(stats, caches, block_ids, p, ref_keep, hashes, hash_layers):
    """Engine keep set against the reference's (near-ties judged on the checker's rows); when the sets are equal, the
    reference's whole-region output hashes must be reproduced too."""
    import numpy as np
    from conftest import tensor_sha
    from golden_cases import stats_by_layer
    from triattention_b200 import kv_compaction
    T, bs, k = p["total_tokens"], p["block_size"], p["budget"]
    ds = device_stats(stats, oracle.geometric_offsets())
    dc = [c.to(DEV) for c in caches]
    view = ops.PagedCacheView.from_layers(dc, kv_axis=0)
    g = p["num_q_heads"] // p["num_kv_heads"]
    bt = block_table_tensor([block_ids])
    layout = view.layout(1, g, bt.shape[1])
    meta = torch.tensor([T, p["round_start"], k, 0], dtype=torch.int32, device=DEV)
    keep = ops.compress_paged(view, layout, ds, bt, meta[0:1], meta[1:2], None, meta[2:3], k, p["window"],
                              status=meta[3:4])[0].cpu().long()
    assert int(meta[3].item()) == 0
    if not torch.equal(keep, ref_keep):
        layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
        fin = oracle.final_scores_group_per_head(layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(),
                                                 T, p["round_start"], window_size=p["window"], kv_axis=0)
        ok, nd = keep_sets_match_modulo_near_ties(keep, ref_keep, fin)
        assert ok, nd
        return False
    # same keep set: the whole region (kept prefix + dropped tail, as the reference writes it) must hash equal
    for l, want in zip(hash_layers, hashes):
        d = caches[l].to(DEV)
        n = kv_compaction.compact_request_kv_in_place_per_head(d, block_ids, bs, ref_keep.to(DEV), T,
                                                               preserve_dropped_tokens=True)
        assert n == k and tensor_sha(d) == want, l
    return True


@pytest.mark.parametrize("name", ["c0_exact", "c1_slice"])
def test_reference_outputs_at_benchmark_shapes(manifest, name):
    import numpy as np
    from conftest import GOLDEN
    from golden_cases import build_paged_case
    z = np.load(GOLDEN / "bench_shape_cases.npz")
    p = manifest["bench_shape_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    ref_keep = torch.from_numpy(z[f"{name}/keep"]).long()
    _device_keep_vs_reference(stats, caches, block_ids, p, ref_keep, p["cache_out_sha256"], range(p["num_layers"]))


def test_reference_outputs_with_shipped_statistics(manifest):
    import numpy as np
    from conftest import GOLDEN
    from golden_cases import build_paged_case, build_stats_case
    z = np.load(GOLDEN / "shipped_stats_cases.npz")
    p = manifest["shipped_stats_cases"]["cases"]["qwen3_8b_all_layers"]
    _, caches, block_ids = build_paged_case(p)
    stats = synth.SyntheticStats(torch.from_numpy(z["qwen3_8b_all_layers/q_mean_real"]),
                                 torch.from_numpy(z["qwen3_8b_all_layers/q_mean_imag"]),
                                 torch.from_numpy(z["qwen3_8b_all_layers/q_abs_mean"]), synth.rope_inv_freq(128, 1e6), 128, "half")
    _device_keep_vs_reference(stats, caches, block_ids, p, torch.from_numpy(z["qwen3_8b_all_layers/keep"]).long(),
                              p["cache_out_sha256_first_last"], (0, p["num_layers"] - 1))
    p = manifest["shipped_stats_cases"]["cases"]["gpt_oss_yarn"]
    inv = torch.from_numpy(z["gpt_oss_yarn/inv_freq"])
    stats = synth.SyntheticStats(torch.from_numpy(z["gpt_oss_yarn/q_mean_real"]), torch.from_numpy(z["gpt_oss_yarn/q_mean_imag"]),
                                 torch.from_numpy(z["gpt_oss_yarn/q_abs_mean"]), inv, 64, "half")
    caches, block_ids = build_stats_case(p, inv)
    _device_keep_vs_reference(stats, caches, block_ids, p, torch.from_numpy(z["gpt_oss_yarn/keep"]).long(),
                              p["cache_out_sha256"], range(p["num_layers"]))


@pytest.mark.parametrize("g,hkv", [(4, 8), (8, 2)])
def test_results_do_not_depend_on_the_batch(g, hkv):
    """A request gives bit-identical keep sets and caches whether it is compressed alone or next to other requests
    (the moments are accumulated so that they do not depend on how the keys were split over CTAs)."""
    L, D = 3, 128
    lens, budget, window = [2176, 9000, 5000, 2176, 300], [2048, 2048, 1024, 2048, 128], 128
    stats, caches, ids, _ = _build_case(L, hkv * g, hkv, D, lens, seed=4242 + g)
    ds = device_stats(stats, oracle.geometric_offsets())
    starts = [t + 17 for t in lens]
    batch = [c.to(DEV) for c in caches]
    res = engine.PagedCompressor(ds, window=window).compress(ops.PagedCacheView.from_layers(batch, kv_axis=0), ids, lens,
                                                             starts, budget)
    assert res.device_status == 0
    keep_b = res.keep.clone()
    solo = [c.to(DEV) for c in caches]
    view = ops.PagedCacheView.from_layers(solo, kv_axis=0)
    comp = engine.PagedCompressor(ds, window=window)
    for b in range(len(lens)):
        r = comp.compress(view, [ids[b]], [lens[b]], [starts[b]], [budget[b]])
        assert r.device_status == 0
        assert torch.equal(r.keep[0, :, :budget[b]], keep_b[b, :, :budget[b]]), b
    assert all(torch.equal(a, b) for a, b in zip(batch, solo))


# ------------------------------------------------------------------------------------------ many CTAs, many launches
@pytest.mark.parametrize("agg,g", [(_native.OFFSETS_MAX, 4), (_native.OFFSETS_MEAN, 4), (_native.OFFSETS_MEAN, 8)])
def test_scorer_is_repeatable_over_many_launches(agg, g):
    """Thousands of CTAs per launch, dozens of launches: no wait may run out (status 0) and every launch must give
    bit-identical raw scores and moments.  The tensor-core scorer for max aggregation hands a tile to warps that
    each take every fourth tile; a warp that got ahead of the copies once read a stage before it was refilled,
    which showed up as a rare wait timeout and scores that differed between launches."""
    L, B, Hkv, D, T = 8, 8, 8, 128, 16384
    nblk = T // BS
    gen = torch.Generator(device=DEV).manual_seed(77)
    cgen = torch.Generator().manual_seed(77)
    caches = [torch.randn((2, B * nblk + 3, BS, Hkv, D), generator=gen, device=DEV, dtype=torch.float32).to(torch.bfloat16)
              for _ in range(L)]
    perm = torch.randperm(B * nblk, generator=cgen)
    ids = [perm[b * nblk:(b + 1) * nblk].tolist() for b in range(B)]
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hkv * g, D, inv, cgen)
    ds = device_stats(stats, oracle.geometric_offsets())
    view = ops.PagedCacheView.from_layers(caches, kv_axis=0)
    bt = block_table_tensor(ids)
    layout = view.layout(B, g, bt.shape[1])
    seq = torch.full((B,), T, dtype=torch.int32, device=DEV)
    rs = torch.full((B,), T + 5, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    w = ops.prep_weights_fused(ds, rs, agg)
    O = int(ds.offsets.numel())
    raw0, mom0 = ops.score_paged(view, layout, bt, seq, w, agg, O, status=status)
    raw0, mom0 = raw0.clone(), mom0.clone()
    for it in range(40):
        raw, mom = ops.score_paged(view, layout, bt, seq, w, agg, O, status=status)
        assert int(status.item()) == 0, f"launch {it}: device status {int(status.item())}"
        assert torch.equal(raw, raw0), f"launch {it}: raw scores differ"
        assert torch.equal(mom, mom0), f"launch {it}: moments differ"


def test_max_aggregation_calls_on_two_streams():
    """The tensor-core scorer for max aggregation keeps its per-layer tensor maps in a ring that is 8 calls deep:
    calls issued alternately on two streams (6 in flight, different caches) must give what the same calls give
    one after the other on one stream."""
    L, B, Hkv, g, D, T = 3, 2, 2, 4, 128, 2048
    nblk = T // BS
    gen = torch.Generator(device=DEV).manual_seed(5)
    cgen = torch.Generator().manual_seed(5)
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hkv * g, D, inv, cgen)
    ds = device_stats(stats, oracle.geometric_offsets())
    O = int(ds.offsets.numel())
    agg = _native.OFFSETS_MAX
    jobs = []
    for j in range(6):
        caches = [torch.randn((2, B * nblk + 2, BS, Hkv, D), generator=gen, device=DEV, dtype=torch.float32)
                  .to(torch.bfloat16) for _ in range(L)]
        perm = torch.randperm(B * nblk, generator=cgen)
        ids = [perm[b * nblk:(b + 1) * nblk].tolist() for b in range(B)]
        view = ops.PagedCacheView.from_layers(caches, kv_axis=0)
        bt = block_table_tensor(ids)
        jobs.append(dict(caches=caches, view=view, bt=bt, layout=view.layout(B, g, bt.shape[1])))
    seq = torch.full((B,), T, dtype=torch.int32, device=DEV)
    rs = torch.full((B,), T + 3, dtype=torch.int32, device=DEV)
    w = ops.prep_weights_fused(ds, rs, agg)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    want = []
    for job in jobs:
        raw, mom = ops.score_paged(job["view"], job["layout"], job["bt"], seq, w, agg, O, status=status)
        want.append((raw.clone(), mom.clone()))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = []
    for j, job in enumerate(jobs):
        st = streams[j % 2]
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            got.append(ops.score_paged(job["view"], job["layout"], job["bt"], seq, w, agg, O, status=status))
    for st in streams:
        st.synchronize()
    assert int(status.item()) == 0
    for j, ((raw, mom), (raw0, mom0)) in enumerate(zip(got, want)):
        assert torch.equal(raw, raw0) and torch.equal(mom, mom0), j
