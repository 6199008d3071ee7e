"""Multi-GPU parity (needs >= 2 CUDA devices; skipped otherwise): tensor-parallel sharding by KV head.

Two NCCL ranks each hold half of the KV heads.  Per-head mode: every rank's keep rows equal the rows the
single-GPU run produces for those heads (no communication).  Layer-shared mode: the score rows cross the ranks -
stored into the owner's slots by the finalize kernel when the layers divide over the ranks (symmetric memory; NCCL
reduce-scatter where that is unavailable), one all-reduce(MAX) otherwise - and both ranks produce the keep set of
the single-GPU run, over two consecutive steps.  NVLS is disabled for the test.
"""
from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _build(seed=77, layers=2):
    import synth
    gen = torch.Generator().manual_seed(seed)
    L, Hq, Hkv, D, bs = layers, 16, 4, 128, 16
    lens = [900, 1500]
    inv = synth.rope_inv_freq(D, 1e6)
    stats = synth.make_stats(L, Hq, D, inv, gen)
    nblk = [(t + bs - 1) // bs for t in lens]
    perm = synth.random_block_ids(sum(nblk), sum(nblk) + 5, gen)
    ids, o = [], 0
    for n in nblk:
        ids.append(perm[o:o + n])
        o += n
    caches = []
    for _ in range(L):
        c = synth.make_paged_layer(sum(nblk) + 5, bs, Hkv, D, kv_axis=0)
        for b, t in enumerate(lens):
            synth.write_tokens_to_paged(c, 0, ids[b], bs, synth.make_rotated_keys(Hkv, t, D, inv, gen),
                                        synth.make_values(Hkv, t, D, gen))
        caches.append(c)
    return stats, caches, ids, lens, inv


def _dstats(stats, dev):
    from triattention_b200 import ops
    offsets = torch.tensor([float(2 ** i) for i in range(17)])
    return ops.DeviceStats(stats.q_mean_real.to(dev), stats.q_mean_imag.to(dev), stats.q_abs_mean.to(dev),
                           torch.ones_like(stats.q_abs_mean).to(dev), stats.inv_freq.to(dev), offsets.to(dev))


def _worker(rank: int, world: int, port: int, q, layers: int = 2):
    import torch.distributed as dist
    from triattention_b200 import engine, ops, tp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        stats, caches, ids, lens, _ = _build(layers=layers)
        budgets, starts = [256, 512], list(lens)
        lo, hi = tp.head_range(4, rank, world)
        local = [c[:, :, :, lo:hi].contiguous().to(dev) for c in caches]     # this rank's KV heads
        full = _dstats(stats, dev)
        shard = tp.shard_stats(full, rank, world)
        view = ops.PagedCacheView.from_layers(local, kv_axis=0)
        res = engine.PagedCompressor(shard, window=32).compress(view, ids, lens, starts, budgets)
        per_head = res.keep.cpu()
        local2 = [c[:, :, :, lo:hi].contiguous().to(dev) for c in caches]
        view2 = ops.PagedCacheView.from_layers(local2, kv_axis=0)
        timings = {}
        res2 = engine.compress_layer_shared(view2, shard, ids, lens, starts, budgets, window=32, timings=timings)
        # a second step on the same buffers (the peer-store form reuses its receive slots), lengths as they are now
        lens2 = [256, 512]
        res3 = engine.compress_layer_shared(view2, shard, [i[:16] for i in [ids[0]]] + [ids[1][:32]], lens2, starts,
                                            [200, 400], window=32)
        print(f"rank {rank} layers {layers}: exchange = {timings['exchange']}; multicast bound: "
              f"{timings.get('multicast_bound')}", flush=True)
        q.put((rank, per_head, res2.keep.cpu(), res.device_status | res2.device_status | res3.device_status,
               [c.cpu() for c in local2], timings["exchange"], res3.keep.cpu()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("layers", [2, 3])  # 2: whole layers per rank (reduce-scatter + all-gather); 3: all-reduce
def test_tp2_matches_single_gpu(layers):
    import torch.multiprocessing as mp
    from triattention_b200 import engine, ops
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, layers)) for r in range(2)]
    for p in procs:
        p.start()
    out = {}
    for _ in procs:
        rank, per_head, shared, status, caches, exchange, shared3 = q.get(timeout=300)
        out[rank] = (per_head.clone(), shared.clone(), status, [c.clone() for c in caches], exchange, shared3.clone())
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    # single-GPU reference run with all heads
    stats, caches, ids, lens, _ = _build(layers=layers)
    budgets, starts = [256, 512], list(lens)
    dev = torch.device("cuda", 0)
    full = _dstats(stats, dev)
    one = [c.to(dev) for c in caches]
    res = engine.PagedCompressor(full, window=32).compress(ops.PagedCacheView.from_layers(one, kv_axis=0), ids, lens,
                                                           starts, budgets)
    one2 = [c.to(dev) for c in caches]
    res2 = engine.compress_layer_shared(ops.PagedCacheView.from_layers(one2, kv_axis=0), full, ids, lens, starts, budgets,
                                        window=32)
    res3 = engine.compress_layer_shared(ops.PagedCacheView.from_layers(one2, kv_axis=0), full,
                                        [ids[0][:16], ids[1][:32]], [256, 512], starts, [200, 400], window=32)
    for rank in (0, 1):
        per_head, shared, status, shard_caches, exchange, shared3 = out[rank]
        assert status == 0
        # whole layers per rank: peer stores (or the NCCL reduce-scatter where symmetric memory is unavailable)
        assert exchange.startswith(("peer stores", "reduce-scatter") if layers == 2 else "all-reduce"), exchange
        assert torch.equal(shared3, res3.keep.cpu())
        assert torch.equal(per_head, res.keep.cpu()[:, 2 * rank: 2 * rank + 2])       # heads of this rank, no collective
        assert torch.equal(shared, res2.keep.cpu())                                   # identical on every rank
        for l in range(len(caches)):
            assert torch.equal(shard_caches[l], one2[l][:, :, :, 2 * rank: 2 * rank + 2].cpu())
