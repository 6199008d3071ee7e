"""Block-table shrink after compression: host mirror of the worker reclaim sync (CPU) and the device rewrite
kernel against layout_engine.truncate_tail_reclaim_group (GPU)."""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from triattention_b200 import layout_engine, worker_reclaim_sync


def _runner(counts, ids, multi_group=False):
    table = SimpleNamespace(num_blocks_per_row=np.array(counts, dtype=np.int32))
    block_table = SimpleNamespace(block_tables=[table]) if multi_group else table
    input_batch = SimpleNamespace(block_table=block_table, req_id_to_index={f"r{i}": i for i in range(len(counts))})
    requests = {f"r{i}": SimpleNamespace(block_ids=([list(x)],)[0]) for i, x in enumerate(ids)}
    return SimpleNamespace(input_batch=input_batch, requests=requests, cache_config=SimpleNamespace(block_size=16)), table


@pytest.mark.parametrize("multi_group", [False, True])
def test_worker_reclaim_shrinks_rows_and_block_id_lists(multi_group):
    runner, table = _runner([10, 5, 8], [range(10), range(20, 25), range(40, 48)], multi_group)
    events = [
        {"status": "applied", "req_id": "r0", "cache_len_after": 33},    # 3 blocks
        {"status": "skipped", "req_id": "r1", "cache_len_after": 16},    # not applied: untouched
        {"status": "applied", "req_id": "r2", "cache_len_after": 4096},  # needs more than it has: untouched
        {"status": "applied", "req_id": "gone", "cache_len_after": 16},  # unknown request
        {"status": "applied", "req_id": "r1", "cache_len_after": 0},     # non-positive length: ignored
    ]
    worker_reclaim_sync.apply_worker_block_reclaim_events(base_runner=runner, events=events)
    assert table.num_blocks_per_row.tolist() == [3, 5, 8]
    assert runner.requests["r0"].block_ids == [[0, 1, 2]]
    assert runner.requests["r1"].block_ids == [list(range(20, 25))]
    assert runner.requests["r2"].block_ids == [list(range(40, 48))]


def test_worker_reclaim_noop_cases(monkeypatch):
    runner, table = _runner([10], [range(10)])
    worker_reclaim_sync.apply_worker_block_reclaim_events(base_runner=runner, events=None)
    worker_reclaim_sync.apply_worker_block_reclaim_events(base_runner=runner, events=[])
    monkeypatch.setenv("TRIATTN_DEBUG_DISABLE_WORKER_RECLAIM_SYNC", "1")
    worker_reclaim_sync.apply_worker_block_reclaim_events(
        base_runner=runner, events=[{"status": "applied", "req_id": "r0", "cache_len_after": 16}])
    assert table.num_blocks_per_row.tolist() == [10]
    monkeypatch.delenv("TRIATTN_DEBUG_DISABLE_WORKER_RECLAIM_SYNC")
    # a runner that owns its block tables directly has nothing to sync
    worker_reclaim_sync.apply_worker_block_reclaim_events(
        base_runner=SimpleNamespace(input_batch=None, block_tables=[object()]),
        events=[{"status": "applied", "req_id": "r0", "cache_len_after": 16}])


@pytest.mark.gpu
@pytest.mark.parametrize("num_reqs,width,bs", [(1, 8, 16), (7, 40, 16), (1500, 12, 8), (64, 2049, 16)])
def test_device_block_table_rewrite_matches_host_truncation(num_reqs, width, bs):
    from triattention_b200 import ops
    gen = torch.Generator().manual_seed(1234 + num_reqs)
    table = torch.randint(1, 1 << 20, (num_reqs, width), generator=gen, dtype=torch.int32)
    before = torch.randint(0, width + 1, (num_reqs,), generator=gen, dtype=torch.int32)
    lens = torch.randint(0, width * bs + 3 * bs, (num_reqs,), generator=gen, dtype=torch.int32)
    exp_table, exp_after, exp_freed = table.clone(), [], []
    for b in range(num_reqs):
        row = table[b, : int(before[b])].tolist()
        kept, removed, _ = layout_engine.truncate_tail_reclaim_group(gid=0, normalized_block_ids=row,
                                                                     cache_len_after=int(lens[b]), block_size=bs)
        exp_after.append(len(kept))
        exp_freed += removed
        exp_table[b, len(kept): int(before[b])] = -1
    d_table = table.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    after, freed, count = ops.rewrite_block_tables(d_table, before.cuda(), lens.cuda(), bs, fill_value=-1, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert after.cpu().tolist() == exp_after
    assert int(count.item()) == len(exp_freed)
    assert freed[: len(exp_freed)].cpu().tolist() == exp_freed
    assert torch.equal(d_table.cpu(), exp_table)
    if len(exp_freed) > 1:
        # a list that is too short is truncated and reported
        d2 = table.cuda()
        _, freed2, count2 = ops.rewrite_block_tables(d2, before.cuda(), lens.cuda(), bs, freed_capacity=len(exp_freed) - 1,
                                                     fill_value=-1, status=status)
        torch.cuda.synchronize()
        assert int(count2.item()) == len(exp_freed)
        assert freed2[: len(exp_freed) - 1].cpu().tolist() == exp_freed[:-1]
        assert int(status.item()) != 0
