"""Tensor-parallel host logic on CPU: two gloo ranks shard heads and agree on the layer-shared keep set."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from triattention_b200 import ops, tp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(11)
        heads, T, k = 8, 500, 64
        scores = torch.randn((heads, T), generator=g)
        scores[:, -16:] = float("inf")
        full = torch.cat([scores, torch.full((heads, 12), float("-inf"))], dim=1)   # t_pad = 512
        lo, hi = tp.head_range(heads, rank, world)
        local = full[lo:hi].max(dim=0).values.clone()
        tp.allreduce_shared_scores(local)
        keep = oracle.topk_lowest_index(local[:T], k)
        ref = oracle.topk_lowest_index(scores.max(dim=0).values, k)
        # the reduce-scatter form: 4 "layers" of rows, whole layers per rank, top-k on this rank's rows, all-gather
        layers = 4
        rows = torch.stack([full[lo:hi].roll(l, dims=1).max(dim=0).values for l in range(layers)])   # [layers, t_pad]
        same = None
        if tp.can_scatter_rows(layers):
            try:
                mine = tp.reduce_scatter_shared_scores(rows)
                keep_mine = torch.stack([oracle.topk_lowest_index(r[:T], k) for r in mine]).int()
                keep_all = tp.all_gather_keep(keep_mine)
                ref_all = torch.stack([oracle.topk_lowest_index(full.roll(l, dims=1).max(dim=0).values[:T], k)
                                       for l in range(layers)]).int()
                same = bool(torch.equal(keep_all, ref_all))
            except RuntimeError as exc:   # a backend without reduce_scatter_tensor: the all-reduce form stays in use
                same = f"unsupported:{type(exc).__name__}"
        q.put((rank, bool(torch.equal(keep, ref)), (lo, hi), same))
    finally:
        dist.destroy_process_group()


def test_layer_shared_keep_is_identical_on_every_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [o[:3] for o in out] == [(0, True, (0, 4)), (1, True, (4, 8))]
    # gloo may lack reduce_scatter_tensor; where it has it the scattered form must give the reference keep rows
    assert all(o[3] is True or (isinstance(o[3], str) and o[3].startswith("unsupported")) for o in out), out


def test_head_ranges_and_stat_sharding():
    assert tp.head_range(8, 3, 4) == (6, 8)
    with pytest.raises(ValueError):
        tp.head_range(8, 0, 3)
    with pytest.raises(ValueError):
        tp.head_range(8, 4, 4)
    st = ops.DeviceStats(*(torch.arange(2 * 32 * 4, dtype=torch.float32).view(2, 32, 4) for _ in range(4)),
                         torch.ones(4), torch.ones(17))
    sh = tp.shard_stats(st, 1, 8)
    assert sh.num_heads == 4 and torch.equal(sh.q_mean_real, st.q_mean_real[:, 4:8])
    # single process: the all-reduce is a no-op
    x = torch.randn(3, 5)
    assert tp.allreduce_shared_scores(x) is x
