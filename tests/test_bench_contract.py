"""The benchmark's command-line contract, as far as it can be checked without a GPU: the reference arm runs on
the host cores and prints one JSON line with the agreed keys; the product arm refuses to run without a CUDA device
(there is no CPU fallback to measure by mistake)."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

REPO = Path(__file__).resolve().parent.parent


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, str(REPO / "bench.py"), *args], capture_output=True, text=True, timeout=timeout,
                          cwd=str(REPO))


def test_reference_arm_prints_the_contract_line():
    res = _run("--impl", "reference", "--config", "c0", "--steps", "1", "--warmup", "0")
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "config",
                "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["value"] > 0 and line["unit"] == "keys/s" and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["e2e"]["value"] == line["value"]


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a box without a GPU")
def test_product_arm_needs_a_cuda_device():
    res = _run("--config", "c0", "--steps", "1", "--warmup", "0")
    assert res.returncode != 0
    assert "CUDA device" in (res.stderr + res.stdout)
