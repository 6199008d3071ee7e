"""The C-ABI library builds, loads and exports every symbol include/triattn_b200.h declares (no GPU needed)."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

from triattention_b200 import _native, build

REPO = Path(__file__).resolve().parent.parent


def _declared_symbols():
    text = (REPO / "include" / "triattn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(triattn_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build_library()
    assert path.exists()
    lib = ctypes.CDLL(str(path))
    declared = _declared_symbols()
    assert declared, "no declarations found in the header"
    for sym in declared:
        assert hasattr(lib, sym), f"{sym} declared in include/triattn_b200.h but not exported"
    assert sorted(_native.EXPORTED_SYMBOLS) == declared


def test_host_only_queries():
    lib = _native.load()
    assert lib.triattn_abi_version() == _native.ABI_VERSION == 2
    assert _native.status_string(0) == "ok"
    assert [lib.triattn_padded_group(g) for g in (0, 1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 64, 65)] == [0, 1, 2, 4, 4, 8, 8, 8, 12, 12, 16, 64, 0]
    assert lib.triattn_weight_rows(_native.OFFSETS_MEAN, 17) == 3
    assert lib.triattn_weight_rows(_native.OFFSETS_MAX, 17) == 35
    assert lib.triattn_prep_scratch_floats(8, 64, 17, _native.OFFSETS_MEAN) == 8 * 2 * 64
    lay = _native.PagedLayout(num_layers=36, num_reqs=8, num_kv_heads=8, group_size=4, head_dim=128, block_size=16,
                              num_blocks=20000, max_blocks_per_req=2048, block_stride=16 * 8 * 128,
                              token_stride=8 * 128, head_stride=128)
    ws = lib.triattn_compress_workspace_bytes(ctypes.byref(lay), 17, 0, 2048)
    raw_bytes = 36 * 8 * 8 * 32768 * 4 * 4
    assert raw_bytes < ws < raw_bytes * 1.1
    ws_min = lib.triattn_compress_workspace_bytes_min(ctypes.byref(lay), 17, 0, 2048)
    assert ws - ws_min == raw_bytes // 36 * 35 and raw_bytes // 36 < ws_min < raw_bytes // 36 + 32 * 2 ** 20
    assert lib.triattn_compact_preserve_scratch_bytes(ctypes.byref(lay), 100) == 25600 * 2 * 36 * 8 * 8
    bad = _native.PagedLayout(num_layers=0)
    assert lib.triattn_compress_workspace_bytes(ctypes.byref(bad), 17, 0, 2048) == 0
