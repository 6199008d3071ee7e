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


def _append_to_sink(sink_dir: Optional[str], line: str) -> None:
    if not sink_dir:
        return
    try:
        d = Path(sink_dir)
        d.mkdir(parents=True, exist_ok=True)
        with (d / f"triattn_perf_{os.getpid()}.log").open("a", encoding="utf-8") as fp:
            fp.write(line + "\n")
    except OSError:
        pass


_STEP_PHASES = ("total", "state", "compress", "reclaim", "override_prep", "base_exec")


@dataclass
class TriAttentionPerfProfile:
    """Whole model-runner steps, as the worker's runner proxy (``worker_runner.TriAttentionModelRunner``) times them:
    same switches, same counters and the same ``TRIATTN_PERF`` line as the reference's profile
    (runtime/perf_profile.py:31-161) - steps, steps with a trigger / with overrides, compression calls by outcome,
    average milliseconds per phase, the five commonest skip reasons, CUDA-graph modes seen on the outputs."""

    logger: logging.Logger
    enabled: bool = False
    log_every_steps: int = 200
    sink_dir: Optional[str] = None
    total_steps: int = 0
    steps_with_trigger: int = 0
    steps_with_overrides: int = 0
    compress_calls: int = 0
    compress_applied: int = 0
    compress_skipped: int = 0
    compress_errors: int = 0
    phase_ms: dict = field(default_factory=lambda: {p: 0.0 for p in _STEP_PHASES})
    skip_reasons: Counter = field(default_factory=Counter)
    cudagraph_modes: Counter = field(default_factory=Counter)

    @classmethod
    def from_env(cls, logger: logging.Logger) -> "TriAttentionPerfProfile":
        try:
            every = int(os.environ.get("TRIATTN_RUNTIME_PERF_LOG_EVERY", "200"))
        except Exception:
            every = 200
        return cls(logger=logger, enabled=_env_enabled("TRIATTN_RUNTIME_PERF_PROFILE"), log_every_steps=max(1, every),
                   sink_dir=os.environ.get("TRIATTN_RUNTIME_PERF_SINK_DIR"))

    def record_step(self, *, has_trigger: bool, uses_overrides: bool, t_state_ms: float, t_compress_ms: float,
                    t_reclaim_ms: float, t_override_prep_ms: float, t_base_exec_ms: float, t_total_exec_ms: float) -> None:
        if not self.enabled:
            return
        self.total_steps += 1
        self.steps_with_trigger += bool(has_trigger)
        self.steps_with_overrides += bool(uses_overrides)
        for phase, ms in zip(_STEP_PHASES, (t_total_exec_ms, t_state_ms, t_compress_ms, t_reclaim_ms,
                                            t_override_prep_ms, t_base_exec_ms)):
            self.phase_ms[phase] += ms
        if self.total_steps % self.log_every_steps == 0:
            line = self.summary_line()
            self.logger.info("%s", line)
            _append_to_sink(self.sink_dir, line)

    def record_compression_events(self, events: Any) -> None:
        if not self.enabled or not isinstance(events, list):
            return
        for event in events:
            if not isinstance(event, dict):
                continue
            self.compress_calls += 1
            status = str(event.get("status", ""))
            if status == "applied":
                self.compress_applied += 1
            elif status == "error":
                self.compress_errors += 1
            elif status == "skipped":
                self.compress_skipped += 1
                if isinstance(event.get("reason"), str):
                    self.skip_reasons[event["reason"]] += 1

    def record_model_output(self, output: Any) -> None:
        if not self.enabled or output is None:
            return
        try:
            mode = getattr(getattr(output, "cudagraph_stats", None), "runtime_mode", None)
        except Exception:
            return
        if mode is not None:
            self.cudagraph_modes[str(mode)] += 1

    def summary_line(self) -> str:
        n = max(1, self.total_steps)
        avg = " ".join(f"{p}={self.phase_ms[p] / n:.2f}" for p in _STEP_PHASES)
        top = ",".join(f"{r}:{c}" for r, c in self.skip_reasons.most_common(5))
        return (f"TRIATTN_PERF steps={self.total_steps} trig_steps={self.steps_with_trigger} "
                f"override_steps={self.steps_with_overrides} compress_calls={self.compress_calls} "
                f"applied={self.compress_applied} skipped={self.compress_skipped} errors={self.compress_errors} "
                f"avg_ms({avg}) top_skip_reasons={top or 'none'} cudagraph_modes={dict(self.cudagraph_modes)}")
