"""GPU checks at the sizes and shapes of the benchmark configurations.

Small enough for the CPU checker: full parity.  Full-size shapes: size-independent properties (keep rows
strictly ascending and in range, recent window kept, compacted prefix == gather of the original cache by the
keep set, block tables truncated) evaluated with torch on the device.
"""
from __future__ import annotations

import pytest
import torch

import oracle
from gpu_utils import device_stats, keep_sets_match_modulo_near_ties
from triattention_b200 import engine, ops
import synth

pytestmark = pytest.mark.gpu
DEV = "cuda"
BS = 16


def _build(L, Hq, Hkv, D, lens, gen, theta=1e6, llama3=None, kv_axis=0, positions=None):
    inv = synth.rope_inv_freq(D, theta, llama3)
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
        c = synth.make_paged_layer(total, BS, Hkv, D, kv_axis=kv_axis)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, kv_axis, ids[b], BS, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    return stats, caches, ids, inv


def _stats_dict(stats):
    return {l: {"q_mean_real": stats.q_mean_real[l], "q_mean_imag": stats.q_mean_imag[l],
                "q_abs_mean": stats.q_abs_mean[l], "freq_scale_sq": torch.ones_like(stats.q_abs_mean[l])}
            for l in range(stats.num_layers)}


def test_config0_full_size_parity():
    """The single-layer benchmark configuration: 1 layer, 32q/8kv heads, D 128, 4096 tokens at positions 0..4095, query position 4096,
    budget 2048, window 128."""
    gen = torch.Generator().manual_seed(synth.seed_for(0, 0))
    T, budget, window = 4096, 2048, 128
    stats, caches, ids, inv = _build(1, 32, 8, 128, [T], gen)
    ref_final = oracle.final_scores_group_per_head([(0, caches[0], ids[0], BS)], _stats_dict(stats), inv,
                                                   oracle.geometric_offsets(), T, T, window_size=window, kv_axis=0)
    ref_keep = oracle.topk_lowest_index(ref_final, budget)
    dc = [c.to(DEV) for c in caches]
    comp = engine.PagedCompressor(device_stats(stats, oracle.geometric_offsets()), window=window)
    res = comp.compress(ops.PagedCacheView.from_layers(dc, kv_axis=0), ids, [T], [T], [budget])
    assert res.device_status == 0
    keep = res.keep[0].cpu().long()
    ok, nd = keep_sets_match_modulo_near_ties(keep, ref_keep, ref_final)
    assert ok, nd
    exp = caches[0].clone()
    oracle.compact_per_head(exp, ids[0], BS, keep, T, preserve_dropped_tokens=False, kv_axis=0)
    assert torch.equal(dc[0].cpu().view(torch.int16), exp.view(torch.int16))
    assert res.kept_block_ids[0] == ids[0][:128] and res.removed_block_ids[0] == ids[0][128:]


def test_group8_head_dim128_parity():
    """Qwen3-32B head geometry under TP8: 1 local KV head, 8 query heads per KV head, D 128."""
    gen = torch.Generator().manual_seed(synth.seed_for(2, 0))
    T, budget, window = 1500, 512, 128
    stats, caches, ids, inv = _build(2, 8, 1, 128, [T], gen)
    layers = [(l, c, ids[0], BS) for l, c in enumerate(caches)]
    ref_final = oracle.final_scores_group_per_head(layers, _stats_dict(stats), inv, oracle.geometric_offsets(), T, T,
                                                   window_size=window, kv_axis=0)
    dc = [c.to(DEV) for c in caches]
    comp = engine.PagedCompressor(device_stats(stats, oracle.geometric_offsets()), window=window)
    res = comp.compress(ops.PagedCacheView.from_layers(dc, kv_axis=0), ids, [T], [T], [budget])
    assert res.device_status == 0
    ok, nd = keep_sets_match_modulo_near_ties(res.keep[0].cpu().long(), oracle.topk_lowest_index(ref_final, budget), ref_final)
    assert ok, nd


def test_decode_interleaved_rounds_match_checker():
    """Config-3 style: llama3-scaled RoPE, ragged requests, repeated compress -> append -> compress with
    round_start = absolute tokens seen; the device cache and the CPU cache evolve in lockstep."""
    gen = torch.Generator().manual_seed(synth.seed_for(3, 0))
    llama3 = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)
    L, Hq, Hkv, D, budget, window, slack = 2, 8, 2, 128, 256, 32, 32
    lens = [700, 1333, 300]
    inv = synth.rope_inv_freq(D, 5e5, llama3)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    cap = [(max(lens) + 3 * slack + BS) // BS for _ in lens]
    total = sum(cap) + 3
    perm = synth.random_block_ids(sum(cap), total, gen)
    ids, o = [], 0
    for n in cap:
        ids.append(perm[o:o + n])
        o += n
    cpu = [synth.make_paged_layer(total, BS, Hkv, D, kv_axis=0) for _ in range(L)]
    for c in cpu:
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], BS, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
    dev = [c.to(DEV) for c in cpu]
    view = ops.PagedCacheView.from_layers(dev, kv_axis=0)
    comp = engine.PagedCompressor(device_stats(stats, oracle.geometric_offsets()), window=window)
    sd = _stats_dict(stats)
    cur = list(lens)          # tokens currently cached per request
    seen = list(lens)         # absolute tokens computed so far (round_start)
    for rnd in range(3):
        act = [b for b in range(len(lens)) if cur[b] >= budget + slack]
        assert act
        res = comp.compress(view, [ids[b] for b in act], [cur[b] for b in act], [seen[b] for b in act],
                            [budget] * len(act))
        assert res.device_status == 0
        for j, b in enumerate(act):
            layers = [(l, c, ids[b], BS) for l, c in enumerate(cpu)]
            fin = oracle.final_scores_group_per_head(layers, sd, inv, oracle.geometric_offsets(), cur[b], seen[b],
                                                     window_size=window, kv_axis=0)
            keep = res.keep[j].cpu().long()
            ok, nd = keep_sets_match_modulo_near_ties(keep, oracle.topk_lowest_index(fin, budget), fin)
            assert ok, (rnd, b, nd)
            for c in cpu:   # the CPU cache follows the device's keep set so that later rounds stay comparable
                oracle.compact_per_head(c, ids[b], BS, keep, cur[b], preserve_dropped_tokens=False, kv_axis=0)
            cur[b] = budget
        for l in range(L):
            assert torch.equal(dev[l].cpu().view(torch.int16), cpu[l].view(torch.int16)), (rnd, l)
        # decode: every request appends `slack` new tokens at its absolute positions
        for b in range(len(lens)):
            pos = torch.arange(seen[b], seen[b] + slack, dtype=torch.float32)
            for l in range(L):
                k_new = synth.make_rotated_keys(Hkv, slack, D, inv, gen, positions=pos)
                v_new = synth.make_values(Hkv, slack, D, gen)
                tok = torch.arange(cur[b], cur[b] + slack)
                blk = torch.as_tensor(ids[b])[tok // BS]
                cpu[l][0][blk, tok % BS] = k_new
                cpu[l][1][blk, tok % BS] = v_new
                dev[l][0][blk.to(DEV), (tok % BS).to(DEV)] = k_new.to(DEV)
                dev[l][1][blk.to(DEV), (tok % BS).to(DEV)] = v_new.to(DEV)
            cur[b] += slack
            seen[b] += slack


@pytest.mark.parametrize("hkv,g,batch", [(8, 4, 2), (1, 8, 4)])
def test_full_length_properties(hkv, g, batch):
    """32768-token requests (config 1 / config 2 per-GPU head geometry): properties that need no CPU checker."""
    gen = torch.Generator(device=DEV).manual_seed(1234)
    cgen = torch.Generator().manual_seed(1234)
    L, D, T, budget, window = 2, 128, 32768, 2048, 128
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, hkv * g, D, inv, cgen)
    nblk = T // BS
    total = batch * nblk + 5
    perm = torch.randperm(total - 1, generator=cgen)[: batch * nblk] + 1
    ids = [perm[b * nblk:(b + 1) * nblk].tolist() for b in range(batch)]
    caches = [(torch.randn((2, total, BS, hkv, D), generator=gen, device=DEV) * 2).to(torch.bfloat16) for _ in range(L)]
    before = [c.clone() for c in caches]
    comp = engine.PagedCompressor(device_stats(stats, oracle.geometric_offsets()), window=window)
    res = comp.compress(ops.PagedCacheView.from_layers(caches, kv_axis=0), ids, [T] * batch, [T] * batch, [budget] * batch)
    assert res.device_status == 0
    keep = res.keep.long()                                  # [B, Hkv, k]
    assert keep.shape == (batch, hkv, budget)
    assert bool((keep[..., 1:] > keep[..., :-1]).all()) and int(keep.min()) >= 0 and int(keep.max()) < T
    assert bool((keep[..., -window:] == torch.arange(T - window, T, device=DEV)).all())
    hidx = torch.arange(hkv, device=DEV).view(hkv, 1)
    for b in range(batch):
        bt = torch.as_tensor(ids[b], device=DEV)
        src_blk, src_off = bt[keep[b] // BS], keep[b] % BS             # [Hkv, k]
        dst = torch.arange(budget, device=DEV)
        dst_blk, dst_off = bt[dst // BS], dst % BS
        for l in range(L):
            for kv in (0, 1):
                want = before[l][kv][src_blk, src_off, hidx]            # [Hkv, k, D]
                got = caches[l][kv][dst_blk, dst_off].permute(1, 0, 2)  # [Hkv, k, D]
                assert torch.equal(got, want), (b, l, kv)
            # nothing outside the kept prefix of this request changed
            tail = bt[budget // BS:]
            assert torch.equal(caches[l][:, tail], before[l][:, tail])
        assert res.kept_block_ids[b] == ids[b][: budget // BS]
    # idempotence: compressing the compacted prefix with budget == length is the identity
    snap = [c.clone() for c in caches]
    res2 = comp.compress(ops.PagedCacheView.from_layers(caches, kv_axis=0), [i[: budget // BS] for i in ids],
                         [budget] * batch, [T] * batch, [budget] * batch)
    assert bool((res2.keep.long() == torch.arange(budget, device=DEV)).all())
    assert all(torch.equal(a, c) for a, c in zip(snap, caches))


def test_token_pool_layout_block_size_one():
    """A token-granular slot pool (one token per 'block', as a flat KV pool stores it) goes through the same
    entry points: the block table is the request's slot list."""
    gen = torch.Generator().manual_seed(4242)
    L, Hq, Hkv, D, T, budget, window = 2, 4, 2, 128, 333, 100, 16
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    pool = T + 40
    slots = synth.random_block_ids(T, pool, gen)
    caches = []
    for _ in range(L):
        c = torch.zeros((2, pool, 1, Hkv, D), dtype=torch.bfloat16)
        synth.write_tokens_to_paged(c, 0, slots, 1, synth.make_rotated_keys(Hkv, T, D, inv, gen),
                                    synth.make_values(Hkv, T, D, gen))
        caches.append(c)
    layers = [(l, c, slots, 1) for l, c in enumerate(caches)]
    ref_final = oracle.final_scores_group_per_head(layers, _stats_dict(stats), inv, oracle.geometric_offsets(), T, 5000,
                                                   window_size=window, kv_axis=0)
    dc = [c.to(DEV) for c in caches]
    comp = engine.PagedCompressor(device_stats(stats, oracle.geometric_offsets()), window=window)
    res = comp.compress(ops.PagedCacheView.from_layers(dc, kv_axis=0), [slots], [T], [5000], [budget])
    assert res.device_status == 0
    keep = res.keep[0].cpu().long()
    ok, nd = keep_sets_match_modulo_near_ties(keep, oracle.topk_lowest_index(ref_final, budget), ref_final)
    assert ok, nd
    for l, c in enumerate(caches):
        exp = c.clone()
        oracle.compact_per_head(exp, slots, 1, keep, T, preserve_dropped_tokens=False, kv_axis=0)
        assert torch.equal(dc[l].cpu().view(torch.int16), exp.view(torch.int16))
    assert res.kept_block_ids[0] == slots[:budget] and res.removed_block_ids[0] == slots[budget:]


def _check_scorer_against_checker(hkv, g, D, bs, hnd, rope_style, aggregation="mean", cuda_cores=False):
    gen = torch.Generator().manual_seed(synth.seed_for(7, hkv * 100 + g * 10 + (1 if hnd else 0)))
    L, lens = 2, [333, 150, 16]
    Hq = hkv * g
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen, rope_style=rope_style)
    nblk = [(t + bs - 1) // bs for t in lens]
    total = sum(nblk) + 5
    perm = synth.random_block_ids(sum(nblk), total, gen)
    ids, o = [], 0
    for n in nblk:
        ids.append(perm[o:o + n])
        o += n
    caches = []
    for _ in range(L):
        if hnd:
            c = torch.zeros((2, total, hkv, bs, D), dtype=torch.bfloat16).permute(0, 1, 3, 2, 4)
        else:
            c = synth.make_paged_layer(total, bs, hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], bs, synth.make_rotated_keys(hkv, t, D, inv, gen, rope_style=rope_style),
                                        synth.make_values(hkv, t, D, gen))
        caches.append(c)
    dc = [c.to(DEV) for c in caches]
    if hnd:
        dc = [torch.zeros((2, total, hkv, bs, D), dtype=torch.bfloat16, device=DEV).permute(0, 1, 3, 2, 4) for _ in caches]
        for d, c in zip(dc, caches):
            d.copy_(c)
    view = ops.PagedCacheView.from_layers(dc, kv_axis=0)
    width = max(nblk)
    bt = torch.zeros((len(lens), width), dtype=torch.int32)
    for b, row in enumerate(ids):
        bt[b, :len(row)] = torch.tensor(row, dtype=torch.int32)
    bt = bt.to(DEV)
    layout = view.layout(len(lens), g, width, rope_interleaved=rope_style == "interleaved")
    dstats = device_stats(stats, oracle.geometric_offsets())
    seq = torch.tensor(lens, dtype=torch.int32, device=DEV)
    rs = torch.tensor([t + 5 for t in lens], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    from triattention_b200 import _native
    agg = _native.OFFSETS_MAX if aggregation == "max" else _native.OFFSETS_MEAN
    w = ops.prep_weights(dstats, rs, agg)
    try:
        raw, mom = ops.score_paged(view, layout, bt, seq, w, agg, 17, status=status, cuda_cores=cuda_cores)
    except _native.NativeLibraryError as exc:
        if cuda_cores and "unsupported shape" in str(exc):
            pytest.skip("geometry outside the CUDA-core cross-check scorer")
        raise
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for b, t in enumerate(lens):
        layers = [(l, c, ids[b], bs) for l, c in enumerate(caches)]
        _, ref_raws = oracle.final_scores_group_per_head(layers, _stats_dict(stats), inv, oracle.geometric_offsets(), t,
                                                         t + 5, window_size=0, return_raw=True, kv_axis=0,
                                                         rope_style=rope_style, aggregation=aggregation)
        got = raw[:, b, :, :t, :g].permute(0, 1, 3, 2).reshape(L, Hq, t).cpu()
        ref = torch.stack(ref_raws)
        sigma = ref.std(dim=-1, keepdim=True)
        worst = float(((got - ref).abs() / torch.maximum(ref.abs(), sigma).clamp_min(1e-6)).max())
        assert worst <= 1e-3, f"request {b}: raw score error {worst}"  # tolerance of the scores: 1e-3 relative
        m = mom[:, b].cpu()
        assert torch.allclose(m[..., 0], got.double().sum(-1), rtol=1e-6, atol=1e-4)
        assert torch.allclose(m[..., 1], (got.double() ** 2).sum(-1), rtol=1e-6, atol=1e-4)


@pytest.mark.parametrize("score_path", ["mma", "fma"])
@pytest.mark.parametrize("hkv,g,D,bs,hnd,rope_style", [
    (8, 4, 128, 16, False, "half"),        # the benchmark geometry
    (8, 4, 128, 16, True, "half"),         # head-major blocks
    (2, 3, 128, 16, False, "half"),        # odd group size, padded to 4 slots
    (4, 1, 64, 16, False, "half"),         # no grouping, head_dim 64
    (2, 2, 64, 32, True, "interleaved"),   # interleaved RoPE pairs, 32-token head-major blocks
    (1, 6, 128, 16, False, "interleaved"), # 6 query heads per KV head: two column tiles
    (2, 8, 128, 8, False, "half"),         # blocks smaller than a 16-key tile
    (1, 12, 128, 16, False, "half"),       # more than 8 query heads: virtual heads
    (3, 4, 128, 16, False, "half"),        # KV-head count that does not divide the warp count
    (4, 2, 128, 16, False, "half"),        # 4 local KV heads: two cache blocks per stage, reader groups of 4 warps
    (1, 4, 128, 16, True, "half"),         # single-head shard: eight per-warp rings
])
def test_scorer_shape_sweep(hkv, g, D, bs, hnd, rope_style, score_path):
    """Raw scores of both streaming scorers against the checker over head/group/block geometries, ragged lengths."""
    _check_scorer_against_checker(hkv, g, D, bs, hnd, rope_style, cuda_cores=score_path == "fma")


@pytest.mark.parametrize("hkv,g,D,bs,hnd,rope_style", [
    (8, 4, 128, 16, False, "half"),
    (2, 4, 128, 16, True, "half"),
    (2, 3, 64, 32, True, "interleaved"),
    (1, 6, 128, 8, False, "interleaved"),
    (2, 4, 128, 32, False, "interleaved"),  # tcgen05 path: two 16-token boxes per block, interleaved pairs
    (1, 12, 128, 16, False, "half"),        # tcgen05 path: three virtual heads of 4
    (3, 2, 128, 48, True, "half"),          # tcgen05 path: head-major 48-token blocks, half-filled column tiles
])
def test_max_aggregation_scorer_shape_sweep(hkv, g, D, bs, hnd, rope_style):
    """The tensor-core scorer for max aggregation against the checker (one column tile per offset, running max)."""
    _check_scorer_against_checker(hkv, g, D, bs, hnd, rope_style, aggregation="max")
