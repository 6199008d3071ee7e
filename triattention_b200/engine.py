"""Batched compression engine: one native call for all requests that triggered in a step.

The reference compresses one request at a time in a Python loop
(runtime/runner_compression_actions.py:11-237 -> hook_impl.py:59-163) and does
several host synchronisations per layer.  Here the per-step metadata of every
triggered request (block ids, lengths, round starts, budgets) is packed into
one pinned host buffer, copied once, and a single ``triattn_compress_paged``
call scores, selects and compacts all requests and layers; one device->host
read returns the status word.  Block tables are then truncated on the host
exactly like ``truncate_tail_reclaim_group`` (runtime/layout_engine.py:209-227).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from . import _native, ops


@dataclass
class CompressResult:
    """Outcome of one batched compression step."""

    keep: torch.Tensor                     # [B, Hkv, keep_pitch] int32 on device, ascending per row
    keep_counts: list[int]                 # per request: tokens kept (cache_len_after)
    kept_block_ids: list                   # per request: block table after tail truncation
    removed_block_ids: list                # per request: blocks handed back to the allocator
                                           # (lists of int, or int32 array views when arrays were passed in)
    device_status: int                     # 0 or TRIATTN_DEV_* bits
    h2d_bytes: int = 0
    d2h_bytes: int = 0


def num_required_blocks(total_tokens: int, block_size: int) -> int:
    """Blocks needed for ``total_tokens`` (runtime/layout_engine.py:24-27)."""
    if total_tokens <= 0:
        return 0
    return (total_tokens + block_size - 1) // block_size


@dataclass
class PagedCompressor:
    """Score -> select -> compact for a batch of requests of one KV-cache group.

    ``stats`` holds one row of statistics per layer of the group, in the order
    of the layers of the ``PagedCacheView`` passed to :meth:`compress`.
    """

    stats: ops.DeviceStats
    window: int = 128
    normalize: bool = True
    offset_agg: int = _native.OFFSETS_MEAN
    flags: int = 0
    layer_reduce: int = _native.REDUCE_MEAN
    # Replay the step from a CUDA graph once the same geometry (cache group, batch size, table width, keep pitch)
    # has been seen twice: a decode loop compresses the same shapes over and over, and the dozen launches of a
    # small step cost more on the host than on the device.
    use_cuda_graph: bool = False
    # Upper bound on the scratch the step may hold (None: enough to score all layers in one launch).  A worker
    # whose HBM went to the KV pool can cap it; the step is then cut into chunks of as many layers as fit (at
    # least one) and the results stay bit-identical.
    max_workspace_bytes: Optional[int] = None
    _workspace: Optional[torch.Tensor] = field(default=None, repr=False)
    _staging: Optional[torch.Tensor] = field(default=None, repr=False)
    _dev_meta: Optional[torch.Tensor] = field(default=None, repr=False)
    _status_host: Optional[torch.Tensor] = field(default=None, repr=False)
    _graphs: dict = field(default_factory=dict, repr=False)
    _seen: set = field(default_factory=set, repr=False)

    def _buffers(self, n_ints: int, ws_bytes: int, device: torch.device):
        if self._staging is None or self._staging.numel() < n_ints:
            self._staging = torch.empty(n_ints, dtype=torch.int32).pin_memory()
            self._dev_meta = torch.empty(n_ints, dtype=torch.int32, device=device)
            self._graphs.clear()  # captured graphs hold the old buffer addresses
        if self._workspace is None or self._workspace.numel() < ws_bytes:
            self._workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
            self._graphs.clear()
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()

    def compress(
        self,
        view: ops.PagedCacheView,
        block_ids: Sequence[Sequence[int]],
        seq_lens: Sequence[int],
        round_starts: Sequence[int],
        budgets: Sequence[int],
        prefill_lens: Optional[Sequence[int]] = None,
    ) -> CompressResult:
        """Compress every listed request in place; returns keep sets and the truncated block tables.

        ``budgets[b]`` is the number of tokens request ``b`` keeps (``min(budget_total, T)`` of
        hook_runtime_context.py:187); ``prefill_lens`` guards tokens ``< prefill_lens[b]`` when given.
        """
        B = len(block_ids)
        if not (B == len(seq_lens) == len(round_starts) == len(budgets)) or B == 0:
            raise ValueError("block_ids, seq_lens, round_starts and budgets must be non-empty and of equal length")
        bs = view.block_size
        seq_np = np.asarray(seq_lens, dtype=np.int64)
        need_np = np.where(seq_np > 0, (seq_np + bs - 1) // bs, 0)
        have_np = np.fromiter((len(ids) for ids in block_ids), dtype=np.int64, count=B)
        if (need_np > have_np).any():
            b = int(np.argmax(need_np > have_np))
            raise IndexError(f"token indices require block_idx={int(need_np[b]) - 1}, but only {int(have_np[b])} blocks exist")
        g, rem = divmod(self.stats.num_heads, view.num_kv_heads)
        if rem or g <= 0:
            raise RuntimeError(
                f"{_native.TRITON_SCORING_REQUIRED_MARKER}:incompatible_head_mapping:"
                f"source={self.stats.num_heads},target={view.num_kv_heads}")
        if self.stats.num_layers != view.num_layers:
            raise ValueError(f"stats cover {self.stats.num_layers} layers, the cache group has {view.num_layers}")
        max_blocks = int(need_np.max())
        kc_np = np.minimum(np.asarray(budgets, dtype=np.int64), seq_np)
        keep_counts = kc_np.tolist()
        keep_pitch = max(int(kc_np.max()), 1)
        layout = view.layout(B, g, max_blocks, rope_interleaved=self.stats.rope_interleaved)
        O = int(self.stats.offsets.numel())
        ws_bytes = ops.compress_workspace_bytes(layout, O, self.offset_agg, keep_pitch)
        if self.max_workspace_bytes is not None:
            ws_bytes = min(ws_bytes, max(int(self.max_workspace_bytes),
                                         ops.compress_workspace_bytes_min(layout, O, self.offset_agg, keep_pitch)))
        keep_bytes = B * view.num_kv_heads * keep_pitch * 4
        # one staging buffer: block table rows, then seq_lens, round_start, keep_counts, prefill_lens, status
        n_ints = B * max_blocks + 4 * B + 4
        self._buffers(n_ints, ws_bytes + keep_bytes + 256, view.device)
        st = self._staging[:n_ints]
        sn = st.numpy()  # the pinned staging buffer, filled through numpy (block ids may be lists or int arrays)
        # block table: one concatenation of the used id prefixes scattered into the padded rows (no per-row writes)
        bt_flat = sn[: B * max_blocks]
        starts = np.cumsum(need_np) - need_np
        total = int(need_np.sum())
        if total == B * max_blocks:
            bt_flat[:] = np.concatenate([np.asarray(ids[:n], dtype=np.int32) for ids, n in zip(block_ids, need_np.tolist())])
        else:
            bt_flat[:] = 0
            dst = np.arange(total, dtype=np.int64) + np.repeat(np.arange(B, dtype=np.int64) * max_blocks - starts, need_np)
            bt_flat[dst] = np.concatenate([np.asarray(ids[:n], dtype=np.int32) for ids, n in zip(block_ids, need_np.tolist())])
        off = B * max_blocks
        sn[off : off + B] = seq_np
        sn[off + B : off + 2 * B] = round_starts
        sn[off + 2 * B : off + 3 * B] = kc_np
        sn[off + 3 * B : off + 4 * B] = prefill_lens if prefill_lens is not None else 0
        sn[off + 4 * B : n_ints] = 0
        dm = self._dev_meta[:n_ints]
        bt = dm[: B * max_blocks].view(B, max_blocks)
        d_seq = dm[off : off + B]
        d_rs = dm[off + B : off + 2 * B]
        d_kc = dm[off + 2 * B : off + 3 * B]
        d_pre = dm[off + 3 * B : off + 4 * B] if prefill_lens is not None else None
        d_status = dm[off + 4 * B : off + 4 * B + 1]
        ws = self._workspace
        keep = ws[ws_bytes // 256 * 256 + 256 :][:keep_bytes].view(torch.int32).view(B, view.num_kv_heads, keep_pitch)

        def launch():
            dm.copy_(st, non_blocking=True)
            ops.compress_paged(
                view, layout, self.stats, bt, d_seq, d_rs, d_pre, d_kc, keep_pitch, self.window, self.normalize,
                self.offset_agg, self.flags, self.layer_reduce, workspace=ws[:ws_bytes], keep_out=keep, status=d_status)
            self._status_host.copy_(d_status, non_blocking=True)

        if not self.use_cuda_graph:
            launch()
        else:
            # everything the captured launches bake in: cache and statistics addresses, geometry, scoring switches
            sp = self.stats
            key = (int(view.k_ptrs.data_ptr()), int(view.v_ptrs.data_ptr()), view.num_layers, view.num_blocks,
                   view.block_stride, view.token_stride, view.head_stride, B, max_blocks, keep_pitch,
                   prefill_lens is not None, int(st.data_ptr()), int(ws.data_ptr()), int(ws_bytes),
                   int(sp.q_mean_real.data_ptr()), int(sp.q_mean_imag.data_ptr()), int(sp.q_abs_mean.data_ptr()),
                   int(sp.freq_scale_sq.data_ptr()), int(sp.omega.data_ptr()), int(sp.offsets.data_ptr()),
                   bool(sp.rope_interleaved), int(self.window), bool(self.normalize), int(self.offset_agg),
                   int(self.flags), int(self.layer_reduce))
            graph = self._graphs.get(key)
            if graph is not None:
                graph.replay()
            elif key not in self._seen:
                self._seen.add(key)  # first sight: run eagerly (also the warm-up a capture needs)
                launch()
            else:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    launch()
                self._graphs[key] = graph
                graph.replay()  # a capture records, it does not execute
        torch.cuda.current_stream().synchronize()
        status = int(self._status_host[0])
        req_blocks = ((kc_np + bs - 1) // bs).tolist()
        kept = [ids[:r] if isinstance(ids, np.ndarray) else [int(x) for x in ids[:r]] for ids, r in zip(block_ids, req_blocks)]
        removed = [ids[r:] if isinstance(ids, np.ndarray) else [int(x) for x in ids[r:]] for ids, r in zip(block_ids, req_blocks)]
        return CompressResult(keep=keep, keep_counts=keep_counts, kept_block_ids=kept, removed_block_ids=removed,
                              device_status=status, h2d_bytes=n_ints * 4, d2h_bytes=4)


def compress_layer_shared(
    view: ops.PagedCacheView,
    stats: ops.DeviceStats,
    block_ids: Sequence[Sequence[int]],
    seq_lens: Sequence[int],
    round_starts: Sequence[int],
    budgets: Sequence[int],
    window: int = 128,
    normalize: bool = True,
    offset_agg: int = _native.OFFSETS_MEAN,
    flags: int = 0,
    prefill_lens: Optional[Sequence[int]] = None,
    process_group=None,
    reduce_stats_to_kv_heads: bool = True,
    timings: Optional[dict] = None,
) -> CompressResult:
    """Layer-shared selection: every layer keeps ONE token set for all its heads (top-k of the max over heads).

    Follows the reference's opt-in ``per_layer`` mode (selector_hf.py:636-667 with the statistics of each GQA
    group averaged down to its KV head, :147-203) for a batch of requests.  Under tensor parallelism the heads
    of a layer live on different ranks: each rank reduces its local heads, one all-reduce(MAX) over
    ``process_group`` of the fp32 rows ``[L, B, t_pad]`` makes them global, and the deterministic top-k then
    yields the same keep set on every rank.  ``stats`` must already be the rank's shard (``tp.shard_stats``).
    ``process_group=False`` skips the collective even when torch.distributed is initialised (a rank that holds
    all heads).  ``timings``, if given, receives ``allreduce_ms`` (a callable: CUDA-event time of the collectives,
    valid after a synchronize), ``allreduce_bytes`` and ``exchange`` (which form was used: when the layers divide
    over the ranks each rank finishes its own layers only - the finalize kernel stores every row into the owner's
    receive slot over NVLink (``tp.PeerRowExchange``), or a NCCL reduce-scatter moves the rows - followed by a
    top-k on this rank's rows and an all-gather of the keep indices; otherwise one all-reduce).
    Returns keep ``[L, B, keep_pitch]`` (as ``CompressResult.keep``).
    """
    from . import tp as _tp

    B = len(block_ids)
    bs = view.block_size
    dev = view.device
    if reduce_stats_to_kv_heads and stats.num_heads != view.num_kv_heads:
        g0, rem = divmod(stats.num_heads, view.num_kv_heads)
        if rem:
            raise RuntimeError(f"incompatible_head_mapping:source={stats.num_heads},target={view.num_kv_heads}")

        def _avg(x):
            return x.reshape(x.shape[0], view.num_kv_heads, g0, x.shape[-1]).mean(dim=2).contiguous()

        stats = ops.DeviceStats(_avg(stats.q_mean_real), _avg(stats.q_mean_imag), _avg(stats.q_abs_mean),
                                _avg(stats.freq_scale_sq), stats.omega, stats.offsets, stats.rope_interleaved)
    g = stats.num_heads // view.num_kv_heads
    max_blocks = max(num_required_blocks(int(n), bs) for n in seq_lens)
    keep_counts = [min(int(k), int(n)) for k, n in zip(budgets, seq_lens)]
    keep_pitch = max(max(keep_counts), 1)
    bt_host = np.zeros((B, max_blocks), dtype=np.int32)
    for b, ids in enumerate(block_ids):
        nb = num_required_blocks(int(seq_lens[b]), bs)
        if nb > len(ids):
            raise IndexError(f"token indices require block_idx={nb - 1}, but only {len(ids)} blocks exist")
        bt_host[b, :nb] = ids[:nb]
    bt = torch.from_numpy(bt_host).to(dev)
    meta = torch.tensor([list(seq_lens), list(round_starts), keep_counts,
                         list(prefill_lens) if prefill_lens is not None else [0] * B], dtype=torch.int32, device=dev)
    d_seq, d_rs, d_kc, d_pre = meta[0], meta[1], meta[2], meta[3]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    layout = view.layout(B, g, max_blocks, rope_interleaved=stats.rope_interleaved)
    w = ops.prep_weights_fused(stats, d_rs, offset_agg, flags)
    raw, mom = ops.score_paged(view, layout, bt, d_seq, w, offset_agg, int(stats.offsets.numel()), status)
    # max over this rank's KV heads (nothing to reduce with a single local head: the per-head fast kernel serves)
    head_reduce = _native.REDUCE_MAX if view.num_kv_heads > 1 else _native.REDUCE_NONE
    L = view.num_layers
    t_pad = max_blocks * bs
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timings is not None else None
    scatter = process_group is not False and _tp.can_scatter_rows(L, process_group)
    peers = None
    if scatter:
        group = process_group if process_group is not None else None
        peers = _tp.peer_row_exchange(L * B // _tp._group_size(group), t_pad, dev, group)
    fin = None
    if peers is not None:
        # the exchange rides on the finalize: every row goes straight into the slot of the rank that owns its layer
        ops.finalize_scores_scatter(layout, raw, mom, d_seq, d_pre if prefill_lens is not None else None, window,
                                    normalize, _native.REDUCE_MAX, head_reduce, peers.ptrs, peers.rank)
    else:
        fin = ops.finalize_scores(layout, raw, mom, d_seq, d_pre if prefill_lens is not None else None, window,
                                  normalize, _native.REDUCE_MAX, head_reduce, _native.REDUCE_NONE)   # [L, B, 1, t_pad]
        rows = fin.view(L * B, fin.shape[-1])  # rows (l, b)
    if ev:
        ev[0].record()
    if peers is not None:
        peers.barrier()                                    # all ranks' stores into this rank's slots are complete
        slots, folded = peers.views(L * B // peers.world, t_pad)
        mine = ops.max_over_slots(slots, folded)
        if ev:
            ev[1].record()
        keep_mine = ops.select_topk(mine, d_seq, d_kc, B, 1, keep_pitch, status)
        if ev:
            ev[2].record()
        keep = _tp.all_gather_keep(keep_mine, process_group)   # also the barrier that frees the slots for the next step
        if ev:
            ev[3].record()
    elif scatter:
        # whole layers per rank: finished rows of this rank's layers -> top-k on them -> everybody's keep rows
        mine = _tp.reduce_scatter_shared_scores(rows, process_group)
        if ev:
            ev[1].record()
        keep_mine = ops.select_topk(mine, d_seq, d_kc, B, 1, keep_pitch, status)
        if ev:
            ev[2].record()
        keep = _tp.all_gather_keep(keep_mine, process_group)
        if ev:
            ev[3].record()
    else:
        if process_group is not False:
            _tp.allreduce_shared_scores(fin, process_group)
        if ev:
            ev[1].record()
            ev[2].record()
            ev[3].record()
        keep = ops.select_topk(rows, d_seq, d_kc, B, 1, keep_pitch, status)
    if timings is not None:
        timings["allreduce_ms"] = lambda: ev[0].elapsed_time(ev[1]) + ev[2].elapsed_time(ev[3])
        timings["allreduce_bytes"] = L * B * t_pad * 4 + (int(keep.numel()) * 4 if scatter else 0)
        if peers is not None:
            timings["multicast_bound"] = peers.multicast_bound
        timings["exchange"] = (
            "peer stores of the fp32 score rows inside finalize (symmetric memory) + barrier + fold, all-gather of the "
            "keep indices" if peers is not None else
            "reduce-scatter(MAX) of the fp32 score rows + all-gather of the keep indices" if scatter
            else "all-reduce(MAX) of the fp32 score rows")
    ops.compact_paged(view, layout, bt, d_seq, keep, (B * keep_pitch, keep_pitch, 0), d_kc, status)
    bits = int(status.item())
    kept, removed = [], []
    for b, ids in enumerate(block_ids):
        req = num_required_blocks(keep_counts[b], bs)
        kept.append(ids[:req] if isinstance(ids, np.ndarray) else [int(x) for x in ids[:req]])
        removed.append(ids[req:] if isinstance(ids, np.ndarray) else [int(x) for x in ids[req:]])
    return CompressResult(keep=keep.view(L, B, keep_pitch), keep_counts=keep_counts, kept_block_ids=kept,
                          removed_block_ids=removed, device_status=bits, h2d_bytes=bt_host.nbytes + meta.numel() * 4,
                          d2h_bytes=4)
