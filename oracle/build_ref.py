#!/usr/bin/env python
"""Recipe for oracle/_ref: an unmodified copy of the reference's own Python code for this path.

    python oracle/build_ref.py [--reference-root DIR]

TEST / BASELINE INFRASTRUCTURE ONLY.  The reference is pure Python, so "building" it means copying the
packages the score -> select -> compact path imports (triattention/vllm/core, triattention/vllm/runtime,
triattention/common and the package __init__ files) from a checkout of the reference into
``oracle/_ref/triattention``, byte for byte.  ``oracle/_ref`` is ignored by git (nothing of the reference is
committed) but travels with the working tree, so that ``bench.py --impl reference`` and the ``cpu_baseline``
leg can time the reference's OWN CPU code where no checkout is mounted.  Without it they fall back to the
restatement in this package and say so (``kind: "port"``).

Nothing under ``triattention_b200/`` imports this directory.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
SUBTREES = ("triattention/vllm/core", "triattention/vllm/runtime", "triattention/common")
INIT_FILES = ("triattention/__init__.py", "triattention/vllm/__init__.py")


def default_reference_root() -> Path:
    return Path(os.environ.get("TRIATTN_REFERENCE_ROOT", str(HERE.parent.parent / "reference")))


def build(reference_root: Path | None = None, quiet: bool = False) -> Path | None:
    """Copy the reference packages into oracle/_ref; returns the directory, or None when no checkout is present."""
    root = Path(reference_root) if reference_root is not None else default_reference_root()
    if not (root / "triattention" / "vllm" / "core" / "scoring.py").is_file():
        return None
    dst_pkg = REF_DIR / "triattention"
    if dst_pkg.exists():
        shutil.rmtree(dst_pkg)
    digest, n = hashlib.sha256(), 0
    files = [root / f for f in INIT_FILES]
    for sub in SUBTREES:
        files += sorted((root / sub).rglob("*.py"))
    for src in files:
        rel = src.relative_to(root)
        out = REF_DIR / rel
        out.parent.mkdir(parents=True, exist_ok=True)
        data = src.read_bytes()
        out.write_bytes(data)
        digest.update(str(rel).encode() + b"\0" + data)
        n += 1
    (REF_DIR / "MANIFEST.json").write_text(json.dumps(
        {"files": n, "sha256": digest.hexdigest(), "source": "unmodified copy of the reference's Python packages"}, indent=1))
    if not quiet:
        print(f"oracle/_ref: {n} files, sha256 {digest.hexdigest()[:16]}")
    return REF_DIR


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=None)
    args = ap.parse_args()
    if build(args.reference_root) is None:
        sys.exit("no reference checkout found (set TRIATTN_REFERENCE_ROOT or pass --reference-root)")
