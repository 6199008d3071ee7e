"""Torch-tensor wrappers over the C ABI (one function per entry point of include/triattn_b200.h).

PyTorch is used for device memory and streams only; all arithmetic happens in
the CUDA kernels of ``libtriattn_b200.so``.  Every wrapper launches on the
current torch stream and does not synchronise.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _native
from ._native import PagedLayout


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    # raw handle of torch's current stream on the current device (the public current_stream() object costs ~15 us)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def split_kv_axes(kv_cache: torch.Tensor, kv_axis: Optional[int] = None):
    """(key_cache, value_cache) views ``[nb, bs, H, D]`` of a 5-D paged cache.

    Same disambiguation rule as the reference's ``_split_kv_axes``
    (runtime/kv_compaction.py:94-117): the axis of size 2 among the first two
    is the K/V axis; if both are 2 an explicit ``kv_axis`` hint is required.
    """
    if kv_cache.ndim != 5:
        raise ValueError(f"Unsupported kv_cache ndim={kv_cache.ndim}, expect 5")
    d0 = int(kv_cache.shape[0]) == 2
    d1 = int(kv_cache.shape[1]) == 2
    if d0 and d1:
        if kv_axis not in (0, 1):
            raise ValueError(
                "Ambiguous KV layout for compaction: both dim0 and dim1 have size 2. "
                "Register an explicit layout hint via register_kv_layout_axis_hint(...)."
            )
        d0, d1 = kv_axis == 0, kv_axis == 1
    if d0:
        return kv_cache[0], kv_cache[1]
    if d1:
        return kv_cache[:, 0], kv_cache[:, 1]
    raise ValueError("Unsupported KV layout for compaction: expected a dimension with size 2")


_VIEW_CACHE: dict = {}


@dataclass
class PagedCacheView:
    """Device-side description of the layers of one KV-cache group (shared block table)."""

    k_ptrs: torch.Tensor   # [L] int64 on device
    v_ptrs: torch.Tensor   # [L] int64 on device
    num_layers: int
    num_blocks: int
    block_size: int
    num_kv_heads: int
    head_dim: int
    block_stride: int
    token_stride: int
    head_stride: int
    device: torch.device
    dtype: torch.dtype

    @classmethod
    def from_layers(cls, kv_caches: Sequence[torch.Tensor], kv_axis: Optional[int] = None) -> "PagedCacheView":
        if not kv_caches:
            raise ValueError("no kv cache layers")
        # An engine keeps the same cache tensors for its whole life: remember the view (device pointer arrays
        # included) per set of layers, so a compression step costs no per-layer Python and no pointer upload.
        key = (kv_axis, tuple(int(c.data_ptr()) for c in kv_caches), tuple(kv_caches[0].shape),
               tuple(kv_caches[0].stride()), kv_caches[0].dtype, str(kv_caches[0].device))
        hit = _VIEW_CACHE.get(key)
        if hit is not None:
            return hit
        view = cls._build(kv_caches, kv_axis)
        if len(_VIEW_CACHE) >= 64:
            _VIEW_CACHE.clear()
        _VIEW_CACHE[key] = view
        return view

    @classmethod
    def _build(cls, kv_caches: Sequence[torch.Tensor], kv_axis: Optional[int]) -> "PagedCacheView":
        k0, v0 = split_kv_axes(kv_caches[0], kv_axis)
        if k0.dtype not in (torch.bfloat16, torch.float16):
            raise ValueError(f"paged cache must be 16-bit, got {k0.dtype}")
        if k0.dtype != torch.bfloat16:
            raise ValueError("the scorer reads bf16 keys; fp16 caches are not supported")
        if k0.stride(3) != 1:
            raise ValueError("head_dim axis of the paged cache must be contiguous")
        kp, vp = [], []
        for c in kv_caches:
            k, v = split_kv_axes(c, kv_axis)
            if k.shape != k0.shape or k.stride() != k0.stride() or v.stride() != k0.stride():
                raise ValueError("all layers of a KV-cache group must share shape and strides")
            if k.data_ptr() % 16 or v.data_ptr() % 16:
                raise ValueError("paged cache base pointers must be 16-byte aligned")
            kp.append(k.data_ptr())
            vp.append(v.data_ptr())
        dev = k0.device
        return cls(
            k_ptrs=torch.tensor(kp, dtype=torch.int64, device=dev),
            v_ptrs=torch.tensor(vp, dtype=torch.int64, device=dev),
            num_layers=len(kv_caches),
            num_blocks=int(k0.shape[0]),
            block_size=int(k0.shape[1]),
            num_kv_heads=int(k0.shape[2]),
            head_dim=int(k0.shape[3]),
            block_stride=int(k0.stride(0)),
            token_stride=int(k0.stride(1)),
            head_stride=int(k0.stride(2)),
            device=dev,
            dtype=k0.dtype,
        )

    def layout(self, num_reqs: int, group_size: int, max_blocks_per_req: int, rope_interleaved: bool = False) -> PagedLayout:
        return PagedLayout(
            num_layers=self.num_layers, num_reqs=int(num_reqs), num_kv_heads=self.num_kv_heads,
            group_size=int(group_size), head_dim=self.head_dim, block_size=self.block_size,
            num_blocks=self.num_blocks, max_blocks_per_req=int(max_blocks_per_req),
            block_stride=self.block_stride, token_stride=self.token_stride, head_stride=self.head_stride,
            rope_interleaved=1 if rope_interleaved else 0, reserved=0,
        )


@dataclass
class DeviceStats:
    """Calibrated statistics packed for the kernels: ``[L, Hq, F]`` fp32 each, plus omega and offsets."""

    q_mean_real: torch.Tensor
    q_mean_imag: torch.Tensor
    q_abs_mean: torch.Tensor
    freq_scale_sq: torch.Tensor
    omega: torch.Tensor
    offsets: torch.Tensor
    rope_interleaved: bool = False

    @property
    def num_layers(self) -> int:
        return int(self.q_mean_real.shape[0])

    @property
    def num_heads(self) -> int:
        return int(self.q_mean_real.shape[1])

    @property
    def num_freqs(self) -> int:
        return int(self.q_mean_real.shape[2])

    def select_layers(self, layer_indices: Sequence[int]) -> "DeviceStats":
        idx = torch.as_tensor(list(layer_indices), dtype=torch.long, device=self.q_mean_real.device)
        return DeviceStats(
            self.q_mean_real.index_select(0, idx).contiguous(), self.q_mean_imag.index_select(0, idx).contiguous(),
            self.q_abs_mean.index_select(0, idx).contiguous(), self.freq_scale_sq.index_select(0, idx).contiguous(),
            self.omega, self.offsets, self.rope_interleaved)

    def slice_heads(self, start: int, end: int) -> "DeviceStats":
        """Statistics rows of query heads [start, end): the shard a tensor-parallel rank owns."""
        return DeviceStats(
            self.q_mean_real[:, start:end].contiguous(), self.q_mean_imag[:, start:end].contiguous(),
            self.q_abs_mean[:, start:end].contiguous(), self.freq_scale_sq[:, start:end].contiguous(),
            self.omega, self.offsets, self.rope_interleaved)


def _i32(x, device) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x.to(device=device, dtype=torch.int32).contiguous()
    return torch.as_tensor(list(x), dtype=torch.int32, device=device)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise _native.NativeLibraryError(
            f"{_native.TRITON_SCORING_REQUIRED_MARKER}:tensor_not_on_cuda:{name} (there is no CPU path)")


def prep_weights(stats: DeviceStats, round_start: torch.Tensor, offset_agg: int = _native.OFFSETS_MEAN,
                 flags: int = 0) -> torch.Tensor:
    """``[L, B, Hq, rows, F]`` fp32 folded weights (``triattn_prep_weights``)."""
    lib = _native.load()
    _require_cuda(stats.q_mean_real, "stats")
    dev = stats.q_mean_real.device
    rs = _i32(round_start, dev)
    L, Hq, F = stats.num_layers, stats.num_heads, stats.num_freqs
    B, O = int(rs.numel()), int(stats.offsets.numel())
    rows = lib.triattn_weight_rows(offset_agg, O)
    scratch = torch.empty(lib.triattn_prep_scratch_floats(B, F, O, offset_agg), dtype=torch.float32, device=dev)
    out = torch.empty((L, B, Hq, rows, F), dtype=torch.float32, device=dev)
    _native.check(lib.triattn_prep_weights(
        _ptr(stats.q_mean_real), _ptr(stats.q_mean_imag), _ptr(stats.q_abs_mean), _ptr(stats.freq_scale_sq),
        _ptr(stats.omega), _ptr(stats.offsets), _ptr(rs), L, B, Hq, F, O, offset_agg, flags,
        _ptr(scratch), _ptr(out), _stream()), "prep_weights")
    return out


def prep_weights_fused(stats: DeviceStats, round_start: torch.Tensor, offset_agg: int = _native.OFFSETS_MEAN,
                       flags: int = 0, moments_to_clear: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``triattn_prep_weights`` in one launch, no scratch (``triattn_prep_weights_fused``); optionally zeroes
    the ``[L, B, Hq, 2]`` fp64 moments array the scorer accumulates into."""
    lib = _native.load()
    _require_cuda(stats.q_mean_real, "stats")
    dev = stats.q_mean_real.device
    rs = _i32(round_start, dev)
    L, Hq, F = stats.num_layers, stats.num_heads, stats.num_freqs
    B, O = int(rs.numel()), int(stats.offsets.numel())
    out = torch.empty((L, B, Hq, lib.triattn_weight_rows(offset_agg, O), F), dtype=torch.float32, device=dev)
    _native.check(lib.triattn_prep_weights_fused(
        _ptr(stats.q_mean_real), _ptr(stats.q_mean_imag), _ptr(stats.q_abs_mean), _ptr(stats.freq_scale_sq),
        _ptr(stats.omega), _ptr(stats.offsets), _ptr(rs), L, B, Hq, F, O, offset_agg, flags, _ptr(out),
        _ptr(moments_to_clear), _stream()), "prep_weights_fused")
    return out


def score_paged(view: PagedCacheView, layout: PagedLayout, block_table: torch.Tensor, seq_lens: torch.Tensor,
                weights: torch.Tensor, offset_agg: int = _native.OFFSETS_MEAN, num_offsets: int = 17,
                status: Optional[torch.Tensor] = None, raw: Optional[torch.Tensor] = None,
                moments: Optional[torch.Tensor] = None, cuda_cores: bool = False):
    """Raw scores ``[L, B, Hkv, t_pad, Gp]`` fp32 and moments ``[L, B, Hq, 2]`` fp64 (``triattn_score_paged``;
    ``cuda_cores=True`` calls the all-fp32 cross-check ``triattn_score_paged_cuda_cores``)."""
    lib = _native.load()
    gp = lib.triattn_padded_group(layout.group_size)
    if gp == 0:
        _native.check(2, "score_paged:group_size")
    L, B, Hkv = layout.num_layers, layout.num_reqs, layout.num_kv_heads
    t_pad = layout.max_blocks_per_req * layout.block_size
    dev = view.device
    if raw is None:
        raw = torch.empty((L, B, Hkv, t_pad, gp), dtype=torch.float32, device=dev)
    if moments is None:
        moments = torch.empty((L, B, Hkv * layout.group_size, 2), dtype=torch.float64, device=dev)
    fn = lib.triattn_score_paged_cuda_cores if cuda_cores else lib.triattn_score_paged
    _native.check(fn(
        ctypes.byref(layout), _ptr(view.k_ptrs), _ptr(block_table), _ptr(seq_lens), _ptr(weights),
        offset_agg, num_offsets, _ptr(raw), _ptr(moments), _ptr(status), _stream()), "score_paged")
    return raw, moments


def finalize_scores(layout: PagedLayout, raw: torch.Tensor, moments: torch.Tensor, seq_lens: torch.Tensor,
                    prefill_lens: Optional[torch.Tensor], window: int, normalize: bool = True,
                    group_reduce: int = _native.REDUCE_MAX, head_reduce: int = _native.REDUCE_NONE,
                    layer_reduce: int = _native.REDUCE_MEAN) -> torch.Tensor:
    """Scores for the top-k ``[Lo, B, Ho, t_pad]`` fp32 (``triattn_finalize_scores``).

    Entries at or beyond a request's length are not written (left as -inf).
    """
    lib = _native.load()
    L, B, Hkv = layout.num_layers, layout.num_reqs, layout.num_kv_heads
    t_pad = layout.max_blocks_per_req * layout.block_size
    Lo = L if layer_reduce == _native.REDUCE_NONE else 1
    Ho = Hkv if head_reduce == _native.REDUCE_NONE else 1
    dev = raw.device
    out = torch.full((Lo, B, Ho, t_pad), float("-inf"), dtype=torch.float32, device=dev)
    _native.check(lib.triattn_finalize_scores(
        ctypes.byref(layout), _ptr(raw), _ptr(moments), _ptr(seq_lens), _ptr(prefill_lens), int(window),
        1 if normalize else 0, group_reduce, head_reduce, layer_reduce, _ptr(out), _stream()),
        "finalize_scores")
    return out


def finalize_scores_scatter(layout: PagedLayout, raw: torch.Tensor, moments: torch.Tensor, seq_lens: torch.Tensor,
                            prefill_lens: Optional[torch.Tensor], window: int, normalize: bool, group_reduce: int,
                            head_reduce: int, recv_ptrs: torch.Tensor, rank: int) -> None:
    """Per-layer score rows, each stored into the receive buffer of the rank that owns it
    (``triattn_finalize_scores_scatter``).  ``recv_ptrs``: int64 device tensor with one pointer per rank to that
    rank's ``[ranks, rows / ranks, t_pad]`` fp32 buffer, valid on this device (peer mappings; the own buffer
    included)."""
    lib = _native.load()
    _require_cuda(recv_ptrs, "recv_ptrs")
    if recv_ptrs.dtype != torch.int64 or not recv_ptrs.is_contiguous():
        raise ValueError("recv_ptrs must be a contiguous int64 tensor of device pointers")
    _native.check(lib.triattn_finalize_scores_scatter(
        ctypes.byref(layout), _ptr(raw), _ptr(moments), _ptr(seq_lens), _ptr(prefill_lens), int(window),
        1 if normalize else 0, group_reduce, head_reduce, _ptr(recv_ptrs), int(recv_ptrs.numel()), int(rank), _stream()),
        "finalize_scores_scatter")


def max_over_slots(slots: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``slots`` ``[S, ...]`` fp32 -> elementwise maximum over the first axis (``triattn_max_over_slots``)."""
    lib = _native.load()
    _require_cuda(slots, "slots")
    if slots.dtype != torch.float32 or not slots.is_contiguous():
        raise ValueError("slots must be a contiguous fp32 tensor")
    if out is None:
        out = torch.empty(slots.shape[1:], dtype=torch.float32, device=slots.device)
    _native.check(lib.triattn_max_over_slots(_ptr(slots), int(slots.shape[0]), int(out.numel()), _ptr(out), _stream()),
                  "max_over_slots")
    return out


def select_topk(scores: torch.Tensor, seq_lens: torch.Tensor, keep_counts: torch.Tensor, num_reqs: int,
                rows_per_req_inner: int, keep_pitch: int, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ascending keep indices ``[rows, keep_pitch]`` int32 (``triattn_select_topk``); ``scores`` is ``[rows, stride]``."""
    lib = _native.load()
    _require_cuda(scores, "scores")
    rows = int(scores.shape[0])
    if scores.stride(1) != 1:
        raise ValueError("score rows must be contiguous")
    out = torch.empty((rows, keep_pitch), dtype=torch.int32, device=scores.device)
    _native.check(lib.triattn_select_topk(
        _ptr(scores), rows, int(scores.stride(0)), _ptr(seq_lens), _ptr(keep_counts), int(num_reqs),
        int(rows_per_req_inner), _ptr(out), int(keep_pitch), _ptr(status), _stream()), "select_topk")
    return out


def compact_paged(view: PagedCacheView, layout: PagedLayout, block_table: torch.Tensor, seq_lens: torch.Tensor,
                  keep: torch.Tensor, keep_strides: tuple, keep_counts: torch.Tensor,
                  status: Optional[torch.Tensor] = None, preserve_dropped: bool = False,
                  max_dropped_rows: int = 0) -> None:
    """In-place compaction of K and V (``triattn_compact_paged`` / ``triattn_compact_paged_preserve``).

    ``keep_strides`` = (layer, request, head) strides of ``keep`` in elements; 0 shares a row.
    """
    lib = _native.load()
    ls, rs, hs = (int(s) for s in keep_strides)
    if not preserve_dropped:
        _native.check(lib.triattn_compact_paged(
            ctypes.byref(layout), _ptr(view.k_ptrs), _ptr(view.v_ptrs), _ptr(block_table), _ptr(seq_lens),
            _ptr(keep), ls, rs, hs, _ptr(keep_counts), _ptr(status), _stream()), "compact_paged")
        return
    nbytes = lib.triattn_compact_preserve_scratch_bytes(ctypes.byref(layout), int(max_dropped_rows))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=view.device)
    _native.check(lib.triattn_compact_paged_preserve(
        ctypes.byref(layout), _ptr(view.k_ptrs), _ptr(view.v_ptrs), _ptr(block_table), _ptr(seq_lens),
        _ptr(keep), ls, rs, hs, _ptr(keep_counts), int(max_dropped_rows), _ptr(scratch), nbytes, _ptr(status),
        _stream()), "compact_paged_preserve")


def compress_workspace_bytes(layout: PagedLayout, num_offsets: int, offset_agg: int, keep_pitch: int) -> int:
    """Workspace with which the fused step scores all layers in one launch."""
    return int(_native.load().triattn_compress_workspace_bytes(ctypes.byref(layout), num_offsets, offset_agg, keep_pitch))


def compress_workspace_bytes_min(layout: PagedLayout, num_offsets: int, offset_agg: int, keep_pitch: int) -> int:
    """Smallest workspace the fused step accepts (raw scores of one layer at a time)."""
    return int(_native.load().triattn_compress_workspace_bytes_min(ctypes.byref(layout), num_offsets, offset_agg, keep_pitch))


def compress_paged(view: PagedCacheView, layout: PagedLayout, stats: DeviceStats, block_table: torch.Tensor,
                   seq_lens: torch.Tensor, round_start: torch.Tensor, prefill_lens: Optional[torch.Tensor],
                   keep_counts: torch.Tensor, keep_pitch: int, window: int, normalize: bool = True,
                   offset_agg: int = _native.OFFSETS_MEAN, flags: int = 0,
                   layer_reduce: int = _native.REDUCE_MEAN, workspace: Optional[torch.Tensor] = None,
                   keep_out: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The fused default-mode step (``triattn_compress_paged``); returns keep ``[B, Hkv, keep_pitch]`` int32."""
    lib = _native.load()
    O = int(stats.offsets.numel())
    if workspace is None:
        workspace = torch.empty(compress_workspace_bytes(layout, O, offset_agg, keep_pitch), dtype=torch.uint8,
                                device=view.device)
    if keep_out is None:
        keep_out = torch.empty((layout.num_reqs, layout.num_kv_heads, keep_pitch), dtype=torch.int32, device=view.device)
    _native.check(lib.triattn_compress_paged(
        ctypes.byref(layout), _ptr(view.k_ptrs), _ptr(view.v_ptrs), _ptr(block_table), _ptr(seq_lens),
        _ptr(round_start), _ptr(prefill_lens), _ptr(keep_counts), _ptr(stats.q_mean_real), _ptr(stats.q_mean_imag),
        _ptr(stats.q_abs_mean), _ptr(stats.freq_scale_sq), _ptr(stats.omega), _ptr(stats.offsets), O, offset_agg,
        flags, int(window), 1 if normalize else 0, layer_reduce, _ptr(workspace), workspace.numel(),
        _ptr(keep_out), int(keep_pitch), _ptr(status), _stream()), "compress_paged")
    return keep_out


def rewrite_block_tables(block_table: torch.Tensor, blocks_before: torch.Tensor, lens_after: torch.Tensor,
                         block_size: int, freed_capacity: Optional[int] = None, fill_value: int = 0,
                         status: Optional[torch.Tensor] = None):
    """Shrink every row of a device block table to ``ceil(lens_after / block_size)`` entries in place
    (``triattn_rewrite_block_tables``).

    Returns ``(blocks_after [B] int32, freed_ids [capacity] int32, freed_count [1] int32)``, all on the device;
    the freed ids are ordered by request, then by position in the row, like the concatenation of the
    ``removed_block_ids`` lists of layout_engine.truncate_tail_reclaim_group.
    """
    lib = _native.load()
    _require_cuda(block_table, "block_table")
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous int32 [B, max_blocks] tensor")
    B, width = int(block_table.shape[0]), int(block_table.shape[1])
    dev = block_table.device
    cap = B * width if freed_capacity is None else int(freed_capacity)
    blocks_after = torch.empty(B, dtype=torch.int32, device=dev)
    freed = torch.empty(max(cap, 1), dtype=torch.int32, device=dev)
    count = torch.zeros(1, dtype=torch.int32, device=dev)
    _native.check(lib.triattn_rewrite_block_tables(
        _ptr(block_table), B, width, int(block_size), _ptr(blocks_before), _ptr(lens_after), _ptr(blocks_after),
        _ptr(freed), cap, _ptr(count), int(fill_value), _ptr(status), _stream()), "rewrite_block_tables")
    return blocks_after, freed, count
