"""Build libtriattn_b200.so in-tree with nvcc for sm_100a.

    python -m triattention_b200.build [--force]

The library has no dependency besides the CUDA runtime; the Python package
loads it with ctypes (``triattention_b200._native``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libtriattn_b200.so"
SOURCES = ["api.cu"]
HEADERS = ["common.cuh", "prep.cuh", "score.cuh", "score_fma.cuh", "score_mma.cuh", "score_mma_max.cuh", "score_umma_max.cuh", "finalize.cuh", "select.cuh", "compact.cuh", "reclaim.cuh", "overrides.cuh",
           "../../include/triattn_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "shared",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or add it to PATH")
    return cand


# Test-only variant: every bounded wait gives up after about a millisecond and every barrier expects 16 bytes
# more than are ever copied, so the wait-timeout path runs (after all real copies have landed) without any fault.
SHORT_WAIT_LIB_PATH = PKG_DIR.parent / "tests" / "_build" / "libtriattn_b200_shortwait.so"


def is_stale(lib_path: Path = LIB_PATH) -> bool:
    if not lib_path.exists():
        return True
    built = lib_path.stat().st_mtime
    return any((CSRC / f).resolve().stat().st_mtime > built for f in SOURCES + HEADERS)


def build_library(force: bool = False, verbose: bool = False, short_wait: bool = False) -> Path:
    """Compile the CUDA sources into ``libtriattn_b200.so`` (skipped when up to date).

    ``short_wait=True`` builds the test-only variant ``tests/_build/libtriattn_b200_shortwait.so`` instead.
    """
    lib_path = SHORT_WAIT_LIB_PATH if short_wait else LIB_PATH
    if not force and not is_stale(lib_path):
        return lib_path
    lib_path.parent.mkdir(parents=True, exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS, *(["-DTRIATTN_TEST_SHORT_WAIT"] if short_wait else []), "-o", str(lib_path),
           *[str(CSRC / s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return lib_path


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, short_wait="--short-wait" in sys.argv)
    print(path)
