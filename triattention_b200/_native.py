"""ctypes binding of libtriattn_b200.so (the C ABI declared in include/triattn_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or a call
returns a non-zero status, a ``RuntimeError`` carrying the reference's fatal
marker (``TRIATTN_FATAL_TRITON_SCORING_REQUIRED``, runtime/constants.py:3) is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

from .constants import TRITON_SCORING_REQUIRED_MARKER

LIB_NAME = "libtriattn_b200.so"
LIB_PATH = Path(os.environ.get("TRIATTN_B200_LIB") or (Path(__file__).resolve().parent / LIB_NAME))

OK = 0
ABI_VERSION = 2
ERR_LIMIT_EXCEEDED = 6
NOALLOC_PREP_SCRATCH_FLOATS = 65536
OFFSETS_MEAN, OFFSETS_MAX = 0, 1
REDUCE_NONE, REDUCE_MEAN, REDUCE_MAX = 0, 1, 2
FLAG_DISABLE_MLR, FLAG_DISABLE_TRIG = 0x1, 0x2
DEV_BAD_BLOCK_ID, DEV_BAD_KEEP_INDEX, DEV_WAIT_TIMEOUT, DEV_BAD_LENGTH = 0x1, 0x2, 0x4, 0x8

# every symbol include/triattn_b200.h declares
EXPORTED_SYMBOLS = (
    "triattn_abi_version",
    "triattn_status_string",
    "triattn_padded_group",
    "triattn_weight_rows",
    "triattn_prep_scratch_floats",
    "triattn_prep_weights",
    "triattn_prep_weights_fused",
    "triattn_prep_weights_noalloc",
    "triattn_score_paged",
    "triattn_score_paged_cuda_cores",
    "triattn_finalize_scores",
    "triattn_finalize_scores_scatter",
    "triattn_max_over_slots",
    "triattn_select_topk",
    "triattn_compact_paged",
    "triattn_compact_preserve_scratch_bytes",
    "triattn_compact_paged_preserve",
    "triattn_compress_workspace_bytes",
    "triattn_compress_workspace_bytes_min",
    "triattn_compress_paged",
    "triattn_rewrite_block_tables",
    "triattn_apply_effective_overrides",
)


class PagedLayout(Structure):
    """Mirror of ``triattn_paged_layout``."""

    _fields_ = [
        ("num_layers", c_int32),
        ("num_reqs", c_int32),
        ("num_kv_heads", c_int32),
        ("group_size", c_int32),
        ("head_dim", c_int32),
        ("block_size", c_int32),
        ("num_blocks", c_int32),
        ("max_blocks_per_req", c_int32),
        ("block_stride", c_int64),
        ("token_stride", c_int64),
        ("head_stride", c_int64),
        ("rope_interleaved", c_int32),
        ("reserved", c_int32),
    ]


_lib = None


class NativeLibraryError(RuntimeError):
    pass


def _declare(lib) -> None:
    P = c_void_p
    LP = POINTER(PagedLayout)
    lib.triattn_abi_version.restype = c_int
    lib.triattn_abi_version.argtypes = []
    lib.triattn_status_string.restype = c_char_p
    lib.triattn_status_string.argtypes = [c_int]
    lib.triattn_padded_group.restype = c_int
    lib.triattn_padded_group.argtypes = [c_int]
    lib.triattn_weight_rows.restype = c_int
    lib.triattn_weight_rows.argtypes = [c_int, c_int]
    lib.triattn_prep_scratch_floats.restype = c_size_t
    lib.triattn_prep_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.triattn_prep_weights.restype = c_int
    lib.triattn_prep_weights.argtypes = [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P]
    lib.triattn_prep_weights_noalloc.restype = c_int
    lib.triattn_prep_weights_noalloc.argtypes = [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P]
    lib.triattn_prep_weights_fused.restype = c_int
    lib.triattn_prep_weights_fused.argtypes = [P, P, P, P, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P, P]
    lib.triattn_score_paged.restype = c_int
    lib.triattn_score_paged.argtypes = [LP, P, P, P, P, c_int, c_int, P, P, P, P]
    lib.triattn_score_paged_cuda_cores.restype = c_int
    lib.triattn_score_paged_cuda_cores.argtypes = [LP, P, P, P, P, c_int, c_int, P, P, P, P]
    lib.triattn_finalize_scores.restype = c_int
    lib.triattn_finalize_scores.argtypes = [LP, P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, P]
    lib.triattn_finalize_scores_scatter.restype = c_int
    lib.triattn_finalize_scores_scatter.argtypes = [LP, P, P, P, P, c_int, c_int, c_int, c_int, P, c_int, c_int, P]
    lib.triattn_max_over_slots.restype = c_int
    lib.triattn_max_over_slots.argtypes = [P, c_int, c_int64, P, P]
    lib.triattn_select_topk.restype = c_int
    lib.triattn_select_topk.argtypes = [P, c_int, c_int64, P, P, c_int, c_int, P, c_int, P, P]
    lib.triattn_compact_paged.restype = c_int
    lib.triattn_compact_paged.argtypes = [LP, P, P, P, P, P, c_int64, c_int64, c_int64, P, P, P]
    lib.triattn_compact_preserve_scratch_bytes.restype = c_size_t
    lib.triattn_compact_preserve_scratch_bytes.argtypes = [LP, c_int]
    lib.triattn_compact_paged_preserve.restype = c_int
    lib.triattn_compact_paged_preserve.argtypes = [LP, P, P, P, P, P, c_int64, c_int64, c_int64, P, c_int, P,
                                                   c_size_t, P, P]
    lib.triattn_compress_workspace_bytes.restype = c_size_t
    lib.triattn_compress_workspace_bytes.argtypes = [LP, c_int, c_int, c_int]
    lib.triattn_compress_workspace_bytes_min.restype = c_size_t
    lib.triattn_compress_workspace_bytes_min.argtypes = [LP, c_int, c_int, c_int]
    lib.triattn_compress_paged.restype = c_int
    lib.triattn_compress_paged.argtypes = [LP, P, P, P, P, P, P, P, P, P, P, P, P, P, c_int, c_int, c_int, c_int,
                                           c_int, c_int, P, c_size_t, P, c_int, P, P]
    lib.triattn_rewrite_block_tables.restype = c_int
    lib.triattn_rewrite_block_tables.argtypes = [P, c_int, c_int, c_int, P, P, P, P, c_int, P, c_int, P, P]
    lib.triattn_apply_effective_overrides.restype = c_int
    lib.triattn_apply_effective_overrides.argtypes = [P, P, c_int, P, P, c_int, P, P, P, c_int, P, c_int, P]


def load():
    """The loaded library (cached).  Raises if it has not been built or lacks a declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryError(
            f"{TRITON_SCORING_REQUIRED_MARKER}:native_library_missing:{LIB_PATH} "
            "(build it with `python -m triattention_b200.build`)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    missing = [s for s in EXPORTED_SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise NativeLibraryError(f"{TRITON_SCORING_REQUIRED_MARKER}:native_symbols_missing:{missing}")
    _declare(lib)
    if lib.triattn_abi_version() != ABI_VERSION:
        raise NativeLibraryError(f"{TRITON_SCORING_REQUIRED_MARKER}:native_abi_mismatch:{lib.triattn_abi_version()}")
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().triattn_status_string(int(status)).decode()


def check(status: int, what: str) -> None:
    """Raise on a non-zero ``triattn_status``."""
    if status != OK:
        raise NativeLibraryError(
            f"{TRITON_SCORING_REQUIRED_MARKER}:native_call_failed:{what}:{status}:{status_string(status)}"
        )
