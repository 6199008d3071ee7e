"""Aggregated timing of the compression hook, gated by the environment.

Keeps the switches and the log-line shape of the reference's worker-side profile
(runtime/perf_profile.py:31-161): ``TRIATTN_RUNTIME_PERF_PROFILE=1`` turns it on,
``TRIATTN_RUNTIME_PERF_LOG_EVERY`` sets the interval (default 200) and ``TRIATTN_RUNTIME_PERF_SINK_DIR``
names a directory that receives ``triattn_perf_<pid>.log``.  The reference aggregates whole model-runner
steps; this package owns only the compression call, so a "step" here is one hook call and the line carries
the fields the hook can know (calls, applied / skipped / errors, average wall time, top skip reasons).
With ``TRIATTN_RUNTIME_NVTX=1`` every hook call is also wrapped in an NVTX range ``triattn.compress``.
"""
from __future__ import annotations

import logging
import os
import time
from collections import Counter
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Optional

_TRUE = {"1", "true", "yes", "on"}


def _env_enabled(name: str) -> bool:
    return str(os.environ.get(name, "0")).strip().lower() in _TRUE


@dataclass
class HookPerfProfile:
    logger: logging.Logger
    enabled: bool = False
    nvtx: bool = False
    log_every: int = 200
    sink_dir: Optional[str] = None
    calls: int = 0
    applied: int = 0
    skipped: int = 0
    errors: int = 0
    t_compress_ms: float = 0.0
    skip_reasons: Counter = field(default_factory=Counter)

    @classmethod
    def from_env(cls, logger: Optional[logging.Logger] = None) -> "HookPerfProfile":
        try:
            every = max(1, int(os.environ.get("TRIATTN_RUNTIME_PERF_LOG_EVERY", "200")))
        except ValueError:
            every = 200
        return cls(logger=logger or logging.getLogger("triattention_b200"),
                   enabled=_env_enabled("TRIATTN_RUNTIME_PERF_PROFILE"), nvtx=_env_enabled("TRIATTN_RUNTIME_NVTX"),
                   log_every=every, sink_dir=os.environ.get("TRIATTN_RUNTIME_PERF_SINK_DIR"))

    def record(self, result: Any, elapsed_ms: float, error: bool = False) -> None:
        self.calls += 1
        self.t_compress_ms += elapsed_ms
        if error:
            self.errors += 1
        elif isinstance(result, dict) and result.get("applied"):
            self.applied += 1
        else:
            self.skipped += 1
            reason = result.get("reason") if isinstance(result, dict) else None
            if isinstance(reason, str):
                self.skip_reasons[reason.split(":")[0]] += 1
        if self.calls % self.log_every == 0:
            self.emit()

    def summary_line(self) -> str:
        n = max(1, self.calls)
        top = ",".join(f"{r}:{c}" for r, c in self.skip_reasons.most_common(5))
        return (f"TRIATTN_PERF steps={self.calls} trig_steps={self.calls} compress_calls={self.calls} "
                f"applied={self.applied} skipped={self.skipped} errors={self.errors} "
                f"avg_ms(compress={self.t_compress_ms / n:.3f}) top_skip_reasons={top or 'none'}")

    def emit(self) -> None:
        line = self.summary_line()
        self.logger.info("%s", line)
        if self.sink_dir:
            try:
                d = Path(self.sink_dir)
                d.mkdir(parents=True, exist_ok=True)
                with (d / f"triattn_perf_{os.getpid()}.log").open("a", encoding="utf-8") as fp:
                    fp.write(line + "\n")
            except OSError:
                pass

    def wrap(self, hook: Callable[..., Any]) -> Callable[..., Any]:
        """``hook`` with timing / NVTX around it; the hook itself when both switches are off."""
        if not (self.enabled or self.nvtx):
            return hook

        def profiled(*args, **kwargs):
            if self.nvtx:
                import torch
                torch.cuda.nvtx.range_push("triattn.compress")
            t0 = time.perf_counter()
            try:
                out = hook(*args, **kwargs)
            except Exception:
                if self.enabled:
                    self.record(None, (time.perf_counter() - t0) * 1e3, error=True)
                raise
            finally:
                if self.nvtx:
                    import torch
                    torch.cuda.nvtx.range_pop()
            if self.enabled:
                self.record(out, (time.perf_counter() - t0) * 1e3)
            return out

        profiled.perf_profile = self  # type: ignore[attr-defined]
        return profiled
