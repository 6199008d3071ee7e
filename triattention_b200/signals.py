"""The per-request message the scheduler sends the worker with every step: trigger decision, the scheduler's cache
length estimate and what the hook needs to interpret it.  Field names, order and defaults are those of the
reference's ``runtime/signals.py:12-26`` (the record is built positionally in places and travels inside the
scheduler output), so the class is generated from one table."""
from __future__ import annotations

import dataclasses
from typing import Literal, Optional

TriggerReason = Literal["none", "length_threshold", "kv_usage_threshold"]

#   name                   type              default        meaning
_SIGNAL_FIELDS = (
    ("req_id",              str,              None),       # request the signal is about
    ("should_compress",     bool,             None),       # compress before this step's forward pass
    ("reason",              TriggerReason,    None),       # which trigger fired ("none" when neither did)
    ("estimated_cache_len", int,              None),       # tokens the cache will hold after this step
    ("step",                int,              None),       # scheduler step counter
    ("kv_usage",            Optional[float],  None),       # KV-pool usage when the pool trigger is enabled
    ("protect_prefill",     bool,             None),       # the prompt is never evicted
    ("prefill_len",         int,              None),       # prompt length
    ("scheduled_tokens",    int,              1),          # tokens of this request in the step (> 1 in a chunked prefill)
)

CompressionSignal = dataclasses.make_dataclass(
    "CompressionSignal",
    [(n, t) if d is None else (n, t, dataclasses.field(default=d)) for n, t, d in _SIGNAL_FIELDS],
    frozen=True, module=__name__)
CompressionSignal.__doc__ = "Compression signal of one request for one scheduler step (immutable)."
