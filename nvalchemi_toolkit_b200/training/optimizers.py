# SPDX-License-Identifier: Apache-2.0
"""Declarative optimiser / scheduler configuration (reference ``nvalchemi/training/optimizers.py:111-447``)."""
from __future__ import annotations

from typing import Any

import torch
from pydantic import BaseModel, ConfigDict, Field

from nvalchemi_toolkit_b200._serialization import import_from_path, type_to_path


class OptimizerConfig(BaseModel):
    """``cls(params, **kwargs)`` plus an optional scheduler.  ``scheduler_metric`` names the validation-summary key fed
    to metric-driven schedulers such as ``ReduceLROnPlateau``."""

    model_config = ConfigDict(arbitrary_types_allowed=True)
    cls: Any = torch.optim.Adam
    kwargs: dict[str, Any] = Field(default_factory=lambda: {"lr": 1e-3})
    scheduler_cls: Any = None
    scheduler_kwargs: dict[str, Any] = Field(default_factory=dict)
    scheduler_metric: str | None = None
    scheduler_interval: str = "step"  # "step" | "epoch" | "validation"

    def build(self, params: Any) -> tuple[torch.optim.Optimizer, Any]:
        cls = import_from_path(self.cls) if isinstance(self.cls, str) else self.cls
        opt = cls(params, **self.kwargs)
        sched = None
        if self.scheduler_cls is not None:
            scls = import_from_path(self.scheduler_cls) if isinstance(self.scheduler_cls, str) else self.scheduler_cls
            sched = scls(opt, **self.scheduler_kwargs)
        return opt, sched

    def to_spec(self) -> dict[str, Any]:
        return {"cls": self.cls if isinstance(self.cls, str) else type_to_path(self.cls), "kwargs": dict(self.kwargs),
                "scheduler_cls": None if self.scheduler_cls is None else (
                    self.scheduler_cls if isinstance(self.scheduler_cls, str) else type_to_path(self.scheduler_cls)),
                "scheduler_kwargs": dict(self.scheduler_kwargs), "scheduler_metric": self.scheduler_metric,
                "scheduler_interval": self.scheduler_interval}


def setup_optimizers(models: dict[str, torch.nn.Module], configs: dict[str, list[OptimizerConfig]],
                     name_filter: set[str] | None = None) -> tuple[list, list, list[str]]:
    """One optimiser (and scheduler slot) per configured (model, config); returns flat lists plus their model keys."""
    opts, scheds, keys = [], [], []
    for key, cfgs in configs.items():
        if key not in models:
            raise KeyError(f"optimizer configured for unknown model '{key}'")
        named = [(n, p) for n, p in models[key].named_parameters() if p.requires_grad]
        if name_filter is not None:
            named = [(n, p) for n, p in named if f"{key}.{n}" in name_filter or n in name_filter]
        for cfg in cfgs if isinstance(cfgs, (list, tuple)) else [cfgs]:
            o, s = cfg.build([p for _, p in named])
            opts.append(o)
            scheds.append(s)
            keys.append(key)
    return opts, scheds, keys


def zero_gradients(opts: list) -> None:
    for o in opts:
        o.zero_grad(set_to_none=True)


def step_optimizers(opts: list) -> None:
    for o in opts:
        o.step()


def step_schedulers(scheds: list, configs: list[OptimizerConfig], interval: str, metrics: dict | None = None) -> None:
    for s, c in zip(scheds, configs):
        if s is None or c.scheduler_interval != interval:
            continue
        if isinstance(s, torch.optim.lr_scheduler.ReduceLROnPlateau):
            if metrics is not None and c.scheduler_metric in metrics:
                s.step(float(metrics[c.scheduler_metric]))
        else:
            s.step()
