"""GPU parity: each C-ABI entry point against the CPU checker and the reference-generated fixtures."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from conftest import np_to_bf16, tensor_sha
from golden_cases import build_paged_case, build_real_stats_case, stats_by_layer
from gpu_utils import (block_table_tensor, device_stats, keep_sets_match_modulo_near_ties, raw_to_reference_layout,
                       score_tolerance_ok)
from triattention_b200 import _native, ops
import synth

pytestmark = pytest.mark.gpu

GROUP_CASES = ["tiny_group", "chunked_group", "c0_like", "llama3_nonorm", "max_agg_prefill", "d64_g8"]


def _agg(p):
    return _native.OFFSETS_MAX if p.get("aggregation", "mean") == "max" else _native.OFFSETS_MEAN


def _oracle_kwargs(p):
    return dict(
        window_size=p["window"], prefill_len=p.get("prefill_len", 0), protect_prefill=p.get("protect_prefill", False),
        normalize=p.get("normalize", True), aggregation=p.get("aggregation", "mean"),
        disable_mlr=p.get("disable_mlr", False), disable_trig=p.get("disable_trig", False),
        rope_style=p.get("rope_style", "half"), kv_axis=p["kv_axis"])


def _run_stages(p, stats, caches, block_ids, cuda_cores=False):
    """prep -> score -> finalize -> select on the device for one request; returns the intermediate tensors."""
    dev = "cuda"
    T, bs = p["total_tokens"], p["block_size"]
    g = p["num_q_heads"] // p["num_kv_heads"]
    dcaches = [c.to(dev) for c in caches]
    view = ops.PagedCacheView.from_layers(dcaches, kv_axis=p["kv_axis"])
    bt = block_table_tensor([block_ids])
    layout = view.layout(1, g, bt.shape[1], rope_interleaved=p.get("rope_style", "half") == "interleaved")
    dstats = device_stats(stats, oracle.geometric_offsets())
    seq = torch.tensor([T], dtype=torch.int32, device=dev)
    rs = torch.tensor([p["round_start"]], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flags = (_native.FLAG_DISABLE_MLR if p.get("disable_mlr") else 0) | (_native.FLAG_DISABLE_TRIG if p.get("disable_trig") else 0)
    w = ops.prep_weights(dstats, rs, _agg(p), flags)
    try:
        raw, mom = ops.score_paged(view, layout, bt, seq, w, _agg(p), 17, status, cuda_cores=cuda_cores)
    except _native.NativeLibraryError as exc:
        if cuda_cores and "unsupported shape" in str(exc):
            pytest.skip("case outside the CUDA-core cross-check scorer (max aggregation or a generic geometry)")
        raise
    pre = None
    if p.get("protect_prefill"):
        pre = torch.tensor([p.get("prefill_len", 0)], dtype=torch.int32, device=dev)
    fin = ops.finalize_scores(layout, raw, mom, seq, pre, p["window"], p.get("normalize", True))
    k = min(p["budget"], T)
    kc = torch.tensor([k], dtype=torch.int32, device=dev)
    keep = ops.select_topk(fin.view(-1, fin.shape[-1]), seq, kc, 1, p["num_kv_heads"], k, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return dict(view=view, layout=layout, bt=bt, seq=seq, kc=kc, raw=raw, mom=mom, fin=fin, keep=keep, caches=dcaches,
                status=status, g=g, dstats=dstats, rs=rs, pre=pre)


@pytest.mark.parametrize("score_path", ["mma", "fma"])
@pytest.mark.parametrize("name", GROUP_CASES)
def test_score_finalize_select_compact_vs_checker(manifest, selector_cases, name, score_path):
    # both streaming scorers (tensor-core default, CUDA-core cross-check) against the same checker and fixtures
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    assert tensor_sha(stats.q_mean_real, stats.q_mean_imag, stats.q_abs_mean, *caches) == p["input_sha256"]
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    ref_final, ref_raws = oracle.final_scores_group_per_head(
        layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"],
        return_raw=True, **_oracle_kwargs(p))
    out = _run_stages(p, stats, caches, block_ids, cuda_cores=score_path == "fma")

    # raw scores: |delta| / max(|ref|, sigma_row) <= 1e-3
    got_raw = raw_to_reference_layout(out["raw"], out["g"], T)[:, 0].cpu()
    ref_raw = torch.stack(ref_raws)
    ok, worst = score_tolerance_ok(got_raw, ref_raw)
    assert ok, f"raw score error {worst}"
    # moments against the double-precision sums of the device's own scores
    mom = out["mom"][:, 0].cpu()
    assert torch.allclose(mom[..., 0], got_raw.double().sum(-1), rtol=1e-6, atol=1e-4)
    assert torch.allclose(mom[..., 1], (got_raw.double() ** 2).sum(-1), rtol=1e-6, atol=1e-4)
    # final scores
    fin = out["fin"][0, 0, :, :T].cpu()
    assert torch.equal(torch.isinf(fin), torch.isinf(ref_final))
    finite = torch.isfinite(ref_final)
    ok, worst = score_tolerance_ok(torch.where(finite, fin, 0.0), torch.where(finite, ref_final, 0.0))
    assert ok, f"final score error {worst}"
    # selection: bit-exact against the checker's top-k on the device's own scores ...
    k = min(p["budget"], T)
    keep = out["keep"].cpu().long()
    assert torch.equal(keep, oracle.topk_lowest_index(fin, k))
    # ... and equal to the reference's keep set except for near-ties at the cut-off
    ref_keep = torch.from_numpy(selector_cases[f"{name}/keep"]).long()
    ok, ndiff = keep_sets_match_modulo_near_ties(keep, ref_keep, ref_final)
    assert ok, f"keep sets differ beyond near-ties ({ndiff} indices)"

    # compaction with the reference's keep set: prefix bit-exact, full region with preserve_dropped
    dev = "cuda"
    keep_ref_dev = ref_keep.to(dev).int().contiguous()
    for preserve in (False, True):
        dc = [c.to(dev) for c in caches]
        view = ops.PagedCacheView.from_layers(dc, kv_axis=p["kv_axis"])
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ops.compact_paged(view, out["layout"], out["bt"], out["seq"], keep_ref_dev, (0, 0, k), out["kc"], status,
                          preserve_dropped=preserve, max_dropped_rows=T - k)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for l, c in enumerate(caches):
            exp = c.clone()
            oracle.compact_per_head(exp, block_ids, bs, ref_keep, T, preserve_dropped_tokens=preserve, kv_axis=p["kv_axis"])
            assert torch.equal(dc[l].cpu().view(torch.int16), exp.view(torch.int16)), f"layer {l} preserve={preserve}"
            if preserve:
                assert tensor_sha(dc[l]) == p["cache_out_sha256"][l]


@pytest.mark.parametrize("name", ["tiny_group", "chunked_group", "c0_like", "d64_g8"])
def test_fused_compress_matches_staged_and_reference(manifest, selector_cases, name):
    p = manifest["selector_cases"]["cases"][name]
    stats, caches, block_ids = build_paged_case(p)
    T, bs = p["total_tokens"], p["block_size"]
    k = min(p["budget"], T)
    out = _run_stages(p, stats, caches, block_ids)
    dev = "cuda"
    dc = [c.to(dev) for c in caches]
    view = ops.PagedCacheView.from_layers(dc, kv_axis=p["kv_axis"])
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    keep = ops.compress_paged(view, out["layout"], out["dstats"], out["bt"], out["seq"], out["rs"], None, out["kc"], k,
                              p["window"], status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(keep[0].cpu(), out["keep"].cpu())
    keep_l = keep[0].cpu().long()
    for l, c in enumerate(caches):
        exp = c.clone()
        oracle.compact_per_head(exp, block_ids, bs, keep_l, T, preserve_dropped_tokens=False, kv_axis=p["kv_axis"])
        assert torch.equal(dc[l].cpu().view(torch.int16), exp.view(torch.int16))


def test_real_stats_case(manifest, real_stats_case):
    p = dict(manifest["real_stats_case"]["params"])
    stats, caches, block_ids = build_real_stats_case(p, real_stats_case)
    T, bs = p["total_tokens"], p["block_size"]
    layers = [(l, c, block_ids, bs) for l, c in enumerate(caches)]
    ref_final = oracle.final_scores_group_per_head(
        layers, stats_by_layer(stats), stats.inv_freq, oracle.geometric_offsets(), T, p["round_start"],
        window_size=p["window"], kv_axis=0)
    out = _run_stages(p, stats, caches, block_ids)
    ref_keep = torch.from_numpy(real_stats_case["keep"]).long()
    ok, ndiff = keep_sets_match_modulo_near_ties(out["keep"].cpu().long(), ref_keep, ref_final)
    assert ok, ndiff


def test_dense_score_variants(manifest, score_cases):
    """Reference scorer outputs for mean/max aggregation, MLR/trig ablations and both RoPE layouts."""
    a = score_cases
    dev = "cuda"
    _, H, T, D = manifest["score_cases"]["shape"]
    for i, v in enumerate(manifest["score_cases"]["variants"]):
        keys = np_to_bf16(a[f"keys_{i}"])[0]  # [H, T, D]
        bs = 16
        nblk = (T + bs - 1) // bs
        cache = torch.zeros((2, nblk + 1, bs, H, D), dtype=torch.bfloat16)
        block_ids = list(range(1, nblk + 1))
        synth.write_tokens_to_paged(cache, 0, block_ids, bs, keys.permute(1, 0, 2), keys.permute(1, 0, 2))
        dcache = cache.to(dev)
        view = ops.PagedCacheView.from_layers([dcache], kv_axis=0)
        bt = block_table_tensor([block_ids])
        layout = view.layout(1, 1, nblk, rope_interleaved=v["rope_style"] == "interleaved")
        st = ops.DeviceStats(
            torch.from_numpy(a["q_mean_real"])[None].to(dev), torch.from_numpy(a["q_mean_imag"])[None].to(dev),
            torch.from_numpy(a["q_abs_mean"])[None].to(dev), torch.from_numpy(a["freq_scale_sq"])[None].to(dev),
            torch.from_numpy(a["omega"]).to(dev), torch.from_numpy(a["offsets"]).to(dev))
        agg = _native.OFFSETS_MAX if v["aggregation"] == "max" else _native.OFFSETS_MEAN
        flags = (_native.FLAG_DISABLE_MLR if v["disable_mlr"] else 0) | (_native.FLAG_DISABLE_TRIG if v["disable_trig"] else 0)
        rs = torch.tensor([v["round_start"]], dtype=torch.int32, device=dev)
        seq = torch.tensor([T], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        w = ops.prep_weights(st, rs, agg, flags)
        raw, _ = ops.score_paged(view, layout, bt, seq, w, agg, 17, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = raw_to_reference_layout(raw, 1, T)[0].cpu()
        ref = torch.from_numpy(a[f"scores_{i}"])
        ok, worst = score_tolerance_ok(got, ref)
        assert ok, f"variant {i} {v}: {worst}"


def test_select_ties_and_edges():
    dev = "cuda"
    g = torch.Generator().manual_seed(3)
    rows, n = 5, 3000
    x = torch.randn((rows, n), generator=g)
    x[0] = 1.0                      # all equal: lowest indices win
    x[1, ::2] = 0.5                 # many ties at the cut-off
    x[1, 1::2] = torch.linspace(-1, 1, n // 2)
    x[2, -128:] = float("inf")      # guard window
    x[3] = torch.round(x[3] * 4) / 4  # heavy quantisation
    x[4, 7] = float("-inf")
    for k in (1, 17, 1024, 2999, 3000, 4000):
        seq = torch.tensor([n], dtype=torch.int32, device=dev)
        kc = torch.tensor([k], dtype=torch.int32, device=dev)
        pitch = max(k, 1)
        keep = ops.select_topk(x.to(dev), seq, kc, 1, rows, pitch)
        torch.cuda.synchronize()
        kk = min(k, n)
        exp = oracle.topk_lowest_index(x, kk)
        assert torch.equal(keep[:, :kk].cpu().long(), exp), k
        if pitch > kk:
            assert bool((keep[:, kk:] == -1).all())


def test_select_ragged_batch():
    dev = "cuda"
    g = torch.Generator().manual_seed(4)
    lens = [100, 5000, 33, 2049]
    ks = [64, 2048, 33, 1]
    heads = 3
    stride = 5008
    x = torch.randn((len(lens), heads, stride), generator=g)
    keep = ops.select_topk(x.view(-1, stride).to(dev), torch.tensor(lens, dtype=torch.int32, device=dev),
                           torch.tensor(ks, dtype=torch.int32, device=dev), len(lens), heads, 2048)
    torch.cuda.synchronize()
    keep = keep.view(len(lens), heads, 2048).cpu().long()
    for b, (n, k) in enumerate(zip(lens, ks)):
        exp = oracle.topk_lowest_index(x[b, :, :n], min(k, n))
        assert torch.equal(keep[b, :, : min(k, n)], exp)


def test_device_status_flags_bad_metadata():
    """Out-of-range block ids and keep indices are reported through the status word; nothing faults."""
    dev = "cuda"
    g = torch.Generator().manual_seed(9)
    T, bs, H, D = 64, 16, 2, 128
    cache = torch.randn((2, 8, bs, H, D), generator=g).to(torch.bfloat16).to(dev)
    view = ops.PagedCacheView.from_layers([cache], kv_axis=0)
    bt = torch.tensor([[1, 2, 99, 3]], dtype=torch.int32, device=dev)  # 99 is out of range
    layout = view.layout(1, 1, 4)
    inv_freq = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(1, H, D, inv_freq, g)
    dstats = device_stats(stats, oracle.geometric_offsets())
    seq = torch.tensor([T], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    w = ops.prep_weights(dstats, torch.tensor([T], dtype=torch.int32, device=dev))
    ops.score_paged(view, layout, bt, seq, w, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & _native.DEV_BAD_BLOCK_ID
    status.zero_()
    bt_ok = torch.tensor([[1, 2, 4, 3]], dtype=torch.int32, device=dev)
    keep = torch.tensor([[[0, 5, 4, 70]] * 1] * H, dtype=torch.int32, device=dev).view(H, 4)  # not ascending, 70 >= T
    before = cache.clone()
    ops.compact_paged(view, layout, bt_ok, seq, keep, (0, 0, 4), torch.tensor([4], dtype=torch.int32, device=dev), status)
    torch.cuda.synchronize()
    assert int(status.item()) & _native.DEV_BAD_KEEP_INDEX
    # valid moves still happened (slot 1 <- token 5), invalid ones were skipped
    kc, _ = ops.split_kv_axes(cache, 0)
    kb, _ = ops.split_kv_axes(before, 0)
    assert torch.equal(kc[1, 1], kb[1, 5])


@pytest.mark.parametrize("preserve", [False, True])
@pytest.mark.parametrize("batch", [1, 40])
def test_compaction_grid_sizes(batch, preserve):
    """Compaction picks its CTA size by the number of (layer, request, head, K/V) streams: a single request runs
    the wide CTAs, 40 requests (640 streams) the narrow ones.  Either way slot r of every stream must hold token
    keep[r], and with ``preserve_dropped`` the dropped tokens follow in ascending order."""
    dev = "cuda"
    g = torch.Generator().manual_seed(77 + batch)
    T, bs, H, D, k = 1000, 16, 8, 128, 333
    nblk = (T + bs - 1) // bs
    total = batch * nblk + 3
    perm = torch.randperm(total - 1, generator=g)[: batch * nblk] + 1
    ids = [perm[b * nblk:(b + 1) * nblk].tolist() for b in range(batch)]
    cache = torch.randn((2, total, bs, H, D), generator=g).to(torch.bfloat16).to(dev)
    before = cache.clone()
    view = ops.PagedCacheView.from_layers([cache], kv_axis=0)
    bt = block_table_tensor(ids)
    layout = view.layout(batch, 1, bt.shape[1])
    keep = torch.stack([torch.stack([torch.randperm(T, generator=g)[:k].sort().values for _ in range(H)])
                        for _ in range(batch)]).to(torch.int32).to(dev)                      # [B, H, k]
    keep[0, 0, :50] = torch.arange(50, dtype=torch.int32)                                   # an unmoved prefix
    keep[0, 0] = keep[0, 0].sort().values
    if int((keep[0, 0, 1:] <= keep[0, 0, :-1]).sum()):                                      # duplicates after the edit
        keep[0, 0] = torch.arange(k, dtype=torch.int32) * 3
    seq = torch.full((batch,), T, dtype=torch.int32, device=dev)
    kc = torch.full((batch,), k, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.compact_paged(view, layout, bt, seq, keep, (0, H * k, k), kc, status, preserve_dropped=preserve,
                      max_dropped_rows=T - k if preserve else 0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    hidx = torch.arange(H, device=dev).view(H, 1)
    for b in range(batch):
        btd = torch.as_tensor(ids[b], device=dev)
        order = keep[b].long()
        if preserve:
            mask = torch.ones((H, T), dtype=torch.bool, device=dev)
            mask[hidx, order] = False
            dropped = torch.arange(T, device=dev).expand(H, T)[mask].view(H, T - k)
            order = torch.cat([order, dropped], dim=1)
        n = order.shape[1]
        dst = torch.arange(n, device=dev)
        for kv in (0, 1):
            want = before[kv][btd[order // bs], order % bs, hidx]                              # [H, n, D]
            got = cache[kv][btd[dst // bs], dst % bs].permute(1, 0, 2)
            assert torch.equal(got, want), (b, kv)
        if not preserve:                                                                       # the tail is untouched
            tail = btd[(k + bs - 1) // bs:]
            assert torch.equal(cache[:, tail], before[:, tail])


def test_abi_rejects_bad_arguments():
    lib = _native.load()
    assert lib.triattn_select_topk(None, 1, 1, None, None, 1, 1, None, 1, None, None) == 1
    lay = _native.PagedLayout(num_layers=1, num_reqs=1, num_kv_heads=1, group_size=80, head_dim=128, block_size=16,
                              num_blocks=4, max_blocks_per_req=4, block_stride=2048, token_stride=128, head_stride=128)
    import ctypes
    x = torch.zeros(16, device="cuda")
    rc = lib.triattn_score_paged(ctypes.byref(lay), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 0, 17,
                                 x.data_ptr(), x.data_ptr(), None, None)
    assert rc == 2  # group size 80 is beyond the supported 64
    with pytest.raises(_native.NativeLibraryError):
        _native.check(rc, "score_paged")


@pytest.mark.parametrize("hkv,g", [(1, 8), (2, 4)])
def test_finalize_scatter_and_max_over_slots(hkv, g):
    """The scattered form of the per-layer finalize: two "ranks" (two sets of raw scores on this device, two receive
    buffers) store their rows into the owner's slots; folding an owner's slots must give, bit for bit, the maximum of
    the two ranks' ordinary finalize outputs for the owner's rows.  One local KV head takes the fast kernel, two (with
    the maximum over heads) the general one."""
    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(41 + hkv)
    L, B, bs, nblk, window = 4, 3, 16, 9, 8
    t_pad = bs * nblk
    gp = _native.load().triattn_padded_group(g)
    layout = _native.PagedLayout(num_layers=L, num_reqs=B, num_kv_heads=hkv, group_size=g, head_dim=128, block_size=bs,
                                 num_blocks=64, max_blocks_per_req=nblk, block_stride=bs * hkv * 128,
                                 token_stride=hkv * 128, head_stride=128, rope_interleaved=0, reserved=0)
    seq = torch.tensor([t_pad, 77, 130], dtype=torch.int32, device=dev)
    pre = torch.tensor([0, 5, 0], dtype=torch.int32, device=dev)
    head_reduce = _native.REDUCE_MAX if hkv > 1 else _native.REDUCE_NONE
    ranks, rows = 2, L * B
    rpr = rows // ranks
    recv = [torch.full((ranks, rpr, t_pad), float("nan"), dtype=torch.float32, device=dev) for _ in range(ranks)]
    ptrs = torch.tensor([r.data_ptr() for r in recv], dtype=torch.int64, device=dev)
    plain = []
    for rank in range(ranks):
        raw = torch.randn((L, B, hkv, t_pad, gp), generator=gen, device=dev)
        n = seq.view(1, B, 1, 1, 1).double()
        valid = (torch.arange(t_pad, device=dev).view(1, 1, 1, t_pad, 1) < seq.view(1, B, 1, 1, 1))
        x = torch.where(valid, raw.double(), torch.zeros((), dtype=torch.float64, device=dev))[..., :g]
        mom = torch.stack([x.sum(3), (x * x).sum(3)], dim=-1).reshape(L, B, hkv * g, 2).contiguous()
        plain.append(ops.finalize_scores(layout, raw, mom, seq, pre, window, True, _native.REDUCE_MAX, head_reduce,
                                         _native.REDUCE_NONE))
        ops.finalize_scores_scatter(layout, raw, mom, seq, pre, window, True, _native.REDUCE_MAX, head_reduce, ptrs, rank)
    torch.cuda.synchronize()
    want = torch.maximum(plain[0], plain[1]).view(rows, t_pad)             # rows (l, b), one head per row
    for owner in range(ranks):
        got = ops.max_over_slots(recv[owner])                               # [rpr, t_pad]
        for i in range(rpr):
            r = owner * rpr + i
            n_tok = int(seq[r % B])
            assert torch.equal(got[i, :n_tok], want[r, :n_tok]), (owner, i)
        # guards arrive as +inf: the last `window` tokens and the protected prompt of request 1
        b1 = [i for i in range(rpr) if (owner * rpr + i) % B == 1][0]
        assert bool(torch.isinf(got[b1, :5]).all()) and bool(torch.isinf(got[b1, 77 - window:77]).all())
    # odd element count: the scalar path of the fold
    x = torch.randn((3, 7), generator=gen, device=dev)
    assert torch.equal(ops.max_over_slots(x), x.max(dim=0).values)
