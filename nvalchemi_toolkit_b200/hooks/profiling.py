# SPDX-License-Identifier: Apache-2.0
"""``TorchProfilerHook``: drives ``torch.profiler`` over a window of steps
(reference ``nvalchemi/hooks/physicsnemo_profiling.py:58-331``; the reference goes through physicsnemo's Profiler)."""
from __future__ import annotations

import os
from enum import Enum
from typing import Any

import torch


class TorchProfilerHook:
    def __init__(self, output_dir: str = "profiler_traces", wait: int = 1, warmup: int = 1, active: int = 3,
                 repeat: int = 1, record_shapes: bool = False, profile_memory: bool = False, with_stack: bool = False,
                 with_flops: bool = False, frequency: int = 1, stage: Enum | None = None) -> None:
        self.output_dir, self.frequency, self.stage = output_dir, frequency, stage
        self.schedule = dict(wait=wait, warmup=warmup, active=active, repeat=repeat)
        self.flags = dict(record_shapes=record_shapes, profile_memory=profile_memory, with_stack=with_stack,
                          with_flops=with_flops)
        self._prof: Any = None

    def on_register(self, owner: Any) -> None:
        if self.stage is None:
            st = getattr(owner, "_stage_type", None)
            self.stage = [s for s in st if s.name in ("AFTER_STEP", "AFTER_BATCH")][0]

    def __enter__(self) -> "TorchProfilerHook":
        rank = int(os.environ.get("RANK", "0"))
        path = os.path.join(self.output_dir, f"rank{rank}")
        os.makedirs(path, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, schedule=torch.profiler.schedule(**self.schedule),
                                            on_trace_ready=torch.profiler.tensorboard_trace_handler(path), **self.flags)
        self._prof.__enter__()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._prof is not None:
            self._prof.__exit__(None, None, None)
            self._prof = None

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if self._prof is not None:
            self._prof.step()
