"""A scripted life of three requests for the request-state store: the fixture generator replays it on the
reference's store, the test on this package's, and the snapshots after every call must agree."""
from __future__ import annotations

import dataclasses

CALLS = [
    ("ensure", dict(req_id="a", prefill_len=100, protect_prefill=False)),
    ("ensure", dict(req_id="b", prefill_len=3000, protect_prefill=True)),
    ("update_cache_len", dict(req_id="a", cache_len=2100, step=1)),
    ("update_cache_len", dict(req_id="zz", cache_len=5, step=1)),
    ("mark_trigger", dict(req_id="a", reason="length_threshold", step=1)),
    ("mark_compressed", dict(req_id="a", step=1, cache_len=2048, scheduled_tokens=1, scheduler_nct=2175)),
    ("ensure", dict(req_id="a", prefill_len=120, protect_prefill=True)),
    ("update_cache_len", dict(req_id="a", cache_len=2100)),
    ("mark_trigger", dict(req_id="b", reason="kv_usage", step=2)),
    ("mark_compression_skipped", dict(req_id="b", reason="prefill_exceeds_budget", step=2)),
    ("mark_compression_skipped", dict(req_id="b", reason="under_budget", step=3)),
    ("mark_preempted", dict(req_id="b")),
    ("ensure", dict(req_id="b", prefill_len=2500, protect_prefill=True)),
    ("mark_resumed", dict(req_id="b")),
    ("mark_compressed", dict(req_id="a", step=9, cache_len=2048)),
    ("mark_compressed", dict(req_id="nobody", step=9, cache_len=1)),
    ("update_cache_len", dict(req_id="a", cache_len=-5, step=10)),
    ("ensure", dict(req_id="c", prefill_len=-7, protect_prefill=False)),
    ("remove", dict(req_id="a")),
    ("remove", dict(req_id="a")),
]


def replay(store) -> list:
    out = []
    for name, kw in CALLS:
        getattr(store, name)(**kw)
        snap = {k: dict(dataclasses.asdict(v), mode=v.mode) for k, v in sorted(store.snapshot().items())}
        out.append({"call": name, "states": snap, "any_compressed": store.has_active_compressed_requests(),
                    "compressed_in_ab": store.has_compressed_request_in(["a", "b"]),
                    "compressed_in_bc": store.has_compressed_request_in(iter(["b", "c"])),
                    "get_a_is_none": store.get("a") is None})
    return out
