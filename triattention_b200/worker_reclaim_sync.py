"""Worker-side block-table shrink after compression (reference: runtime/worker_reclaim_sync.py:15-128).

After a request was compacted to ``cache_len_after`` tokens it needs only
``ceil(cache_len_after / block_size)`` blocks.  The worker's per-row block counters and the per-request block-id
lists are cut to that size so that later appends continue right after the compacted prefix.  Engines that keep
their block tables on the device can do the same for a whole batch with ``ops.rewrite_block_tables``.
"""
from __future__ import annotations

import logging
import os
from typing import Any, Optional

import numpy as np

logger = logging.getLogger(__name__)
_TRUE = {"1", "true", "yes", "on"}
_disabled_logged = False


def _inner_tables(block_table_obj: Any) -> list:
    inner = getattr(block_table_obj, "block_tables", None)   # multi-group table: one inner table per group
    return inner if isinstance(inner, list) else [block_table_obj]


def apply_worker_block_reclaim_events(*, base_runner: Any, events: Optional[list]) -> None:
    """Shrink ``num_blocks_per_row`` and ``req_state.block_ids`` for every applied compression event."""
    global _disabled_logged
    if os.environ.get("TRIATTN_DEBUG_DISABLE_WORKER_RECLAIM_SYNC", "0").strip().lower() in _TRUE:
        if not _disabled_logged:
            logger.info("TriAttention worker reclaim sync disabled by debug env")
            _disabled_logged = True
        return
    if not isinstance(events, list) or not events:
        return
    input_batch = getattr(base_runner, "input_batch", None)
    table_obj = getattr(input_batch, "block_table", None) if input_batch is not None else None
    if table_obj is None:
        if getattr(base_runner, "block_tables", None) is not None:
            return  # runner that owns its tables directly: the hook already updated them
        logger.warning("TriAttention worker reclaim: block table not found")
        return
    row_of = getattr(input_batch, "req_id_to_index", None)
    if not isinstance(row_of, dict):
        logger.warning("TriAttention worker reclaim: req_id_to_index not found on input_batch")
        return
    tables = _inner_tables(table_obj)
    block_size = int(getattr(getattr(base_runner, "cache_config", None), "block_size", 16))
    if block_size <= 0:
        block_size = 16
    requests = getattr(base_runner, "requests", None)
    for event in events:
        if not isinstance(event, dict) or event.get("status") != "applied":
            continue
        req_id = event.get("req_id")
        row = row_of.get(req_id) if req_id is not None else None
        len_after = event.get("cache_len_after")
        if not isinstance(row, int) or not isinstance(len_after, int) or len_after <= 0:
            continue
        need = (len_after + block_size - 1) // block_size
        for table in tables:
            counts = getattr(table, "num_blocks_per_row", None)
            if isinstance(counts, np.ndarray) and int(counts[row]) > need:
                logger.info("TriAttention worker reclaim: req=%s num_blocks %d -> %d", req_id, int(counts[row]), need)
                counts[row] = need
        state = requests.get(req_id) if isinstance(requests, dict) else None
        ids = getattr(state, "block_ids", None) if state is not None else None
        if isinstance(ids, (list, tuple)):
            for group in ids:
                if isinstance(group, list) and len(group) > need:
                    del group[need:]
