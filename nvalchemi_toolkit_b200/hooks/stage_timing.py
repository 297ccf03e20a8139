# SPDX-License-Identifier: Apache-2.0
"""``StageTimingHook``: per-stage timing with CUDA events (or ``perf_counter_ns``), NVTX ranges, CSV and a summary.

Reference: ``nvalchemi/hooks/stage_timing.py:64-476``.  The hook subscribes to every profiled stage, records one
timestamp per stage, and converts timestamps into per-stage durations at the last stage of the step with a single
device synchronisation.  NVTX ranges are pushed through ``torch.cuda.nvtx`` (no extra package needed)."""
from __future__ import annotations

import csv
import time
from enum import Enum
from pathlib import Path
from typing import Any, Literal

import torch


class StageTimingHook:
    def __init__(self, profiled_stages: "set[Enum] | Literal['all', 'step', 'detailed']" = "all", *, frequency: int = 1,
                 enable_nvtx: bool = True, timer_backend: Literal["cuda_event", "perf_counter", "auto"] = "auto",
                 log_path: str | Path | None = None, show_console: bool = False, console_frequency: int = 1,
                 stage: Enum | None = None) -> None:
        self.profiled_stages = profiled_stages
        self.frequency, self.stage = frequency, stage
        self.enable_nvtx = enable_nvtx and torch.cuda.is_available()
        if timer_backend == "auto":
            timer_backend = "cuda_event" if torch.cuda.is_available() else "perf_counter"
        self.timer_backend = timer_backend
        self.log_path = Path(log_path) if log_path is not None else None
        self.show_console, self.console_frequency = show_console, console_frequency
        self._stages: list[Enum] = []
        self._marks: list[tuple[Enum, Any]] = []
        self.rows: list[dict[str, Any]] = []
        self._nvtx_open = False
        self._domain = "dynamics"

    def on_register(self, owner: Any) -> None:
        stage_type = getattr(owner, "_stage_type", None)
        all_stages = list(stage_type) if isinstance(stage_type, type) else []
        if isinstance(self.profiled_stages, set):
            self._stages = sorted(self.profiled_stages, key=lambda s: s.value)
        elif self.profiled_stages == "step" and all_stages:
            self._stages = [all_stages[0], [s for s in all_stages if s.name == "AFTER_STEP"][0]] \
                if any(s.name == "AFTER_STEP" for s in all_stages) else [all_stages[0], all_stages[-1]]
        else:
            self._stages = [s for s in all_stages if s.name != "ON_CONVERGE"]
        self._domain = type(owner).__name__

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in self._stages

    def _now(self) -> Any:
        if self.timer_backend == "cuda_event":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter_ns()

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if self.enable_nvtx:
            if self._nvtx_open:
                torch.cuda.nvtx.range_pop()
            torch.cuda.nvtx.range_push(f"{self._domain}/{stage.name}/{ctx.step_count}")
            self._nvtx_open = True
        self._marks.append((stage, self._now()))
        if stage == self._stages[-1]:
            if self.enable_nvtx and self._nvtx_open:
                torch.cuda.nvtx.range_pop()
                self._nvtx_open = False
            self._finish(ctx.step_count)

    def _finish(self, step: int) -> None:
        marks, self._marks = self._marks, []
        if len(marks) < 2:
            return
        if self.timer_backend == "cuda_event":
            marks[-1][1].synchronize()
        row: dict[str, Any] = {"step": step}
        total = 0.0
        for (s0, t0), (s1, t1) in zip(marks[:-1], marks[1:]):
            ms = t0.elapsed_time(t1) if self.timer_backend == "cuda_event" else (t1 - t0) / 1e6
            row[f"{s0.name}->{s1.name}"] = ms
            total += ms
        row["total_ms"] = total
        self.rows.append(row)
        if self.log_path is not None:
            new = not self.log_path.exists()
            with open(self.log_path, "a", newline="") as f:
                w = csv.DictWriter(f, fieldnames=list(row))
                if new:
                    w.writeheader()
                w.writerow(row)
        if self.show_console and step % self.console_frequency == 0:
            print(" | ".join(f"{k}={v:.3f}" if isinstance(v, float) else f"{k}={v}" for k, v in row.items()))

    def summary(self) -> dict[str, dict[str, float]]:
        """Mean / min / p50 / p99 / max in milliseconds per stage interval."""
        out: dict[str, dict[str, float]] = {}
        keys = [k for k in (self.rows[0] if self.rows else {}) if k != "step"]
        for k in keys:
            v = torch.tensor([r[k] for r in self.rows if k in r], dtype=torch.float64)
            out[k] = {"mean": float(v.mean()), "min": float(v.min()), "p50": float(v.quantile(0.5)),
                      "p99": float(v.quantile(0.99)), "max": float(v.max()), "n": int(v.numel())}
        return out
