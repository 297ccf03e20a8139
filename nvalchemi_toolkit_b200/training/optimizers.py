# SPDX-License-Identifier: Apache-2.0
"""Declarative optimiser / scheduler configuration (reference ``nvalchemi/training/optimizers.py:111-447``)."""
from __future__ import annotations

import inspect
import re
from typing import Any, Callable, Mapping

import torch
from pydantic import BaseModel, ConfigDict, Field, model_validator

from nvalchemi_toolkit_b200._serialization import import_from_path, type_to_path


def check_kwargs(cls: Any, kwargs: Mapping[str, Any], label: str) -> None:
    """Reject keyword arguments the constructor does not accept at configuration time (reference
    ``training/optimizers.py:56-82``): a typo such as ``weight_decy`` should fail when the recipe is read, not after the data
    pipeline and the model are built.  Constructors that take ``**kwargs`` accept everything."""
    try:
        params = inspect.signature(cls.__init__ if isinstance(cls, type) else cls).parameters
    except (TypeError, ValueError):
        return
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
        return
    unknown = sorted(k for k in kwargs if k not in params)
    if unknown:
        accepted = sorted(k for k in params if k not in ("self", "params", "optimizer"))
        raise ValueError(f"{label} {getattr(cls, '__name__', cls)} does not accept {unknown}; accepted: {accepted}")


class ParamGroupSpec(BaseModel):
    """Parameters whose qualified name matches ``pattern`` (``re.search``) form a group with their own optimiser options,
    e.g. ``ParamGroupSpec(pattern=r"bias$|norm", options={"weight_decay": 0.0})`` or a smaller ``lr`` for a pretrained trunk.
    The first matching spec wins; parameters no spec matches use the config's ``kwargs``."""

    pattern: str
    options: dict[str, Any] = Field(default_factory=dict)


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
    #: maps the validation summary to the number a metric-driven scheduler steps on (default: ``summary[scheduler_metric]``)
    scheduler_metric_adapter: Callable[[Mapping[str, Any]], float] | None = None
    param_groups: list[ParamGroupSpec] = Field(default_factory=list)

    @model_validator(mode="after")
    def _validate(self) -> "OptimizerConfig":
        if self.scheduler_interval not in ("step", "epoch", "validation"):
            raise ValueError(f"scheduler_interval must be 'step', 'epoch' or 'validation', got {self.scheduler_interval!r}")
        cls = import_from_path(self.cls) if isinstance(self.cls, str) else self.cls
        check_kwargs(cls, self.kwargs, "optimizer")
        for g in self.param_groups:
            re.compile(g.pattern)
            check_kwargs(cls, g.options, "optimizer (parameter group)")
        if self.scheduler_cls is not None:
            scls = import_from_path(self.scheduler_cls) if isinstance(self.scheduler_cls, str) else self.scheduler_cls
            check_kwargs(scls, self.scheduler_kwargs, "scheduler")
        return self

    def group_parameters(self, named: list[tuple[str, torch.nn.Parameter]]) -> Any:
        """``named`` parameters split into optimiser parameter groups according to ``param_groups``."""
        if not self.param_groups:
            return [p for _, p in named]
        buckets: list[list[torch.nn.Parameter]] = [[] for _ in self.param_groups]
        rest: list[torch.nn.Parameter] = []
        for name, p in named:
            for i, g in enumerate(self.param_groups):
                if re.search(g.pattern, name):
                    buckets[i].append(p)
                    break
            else:
                rest.append(p)
        groups = [{"params": b, **g.options} for b, g in zip(buckets, self.param_groups) if b]
        return ([{"params": rest}] if rest else []) + groups

    def build(self, params: Any) -> tuple[torch.optim.Optimizer, Any]:
        cls = import_from_path(self.cls) if isinstance(self.cls, str) else self.cls
        if params and isinstance(params[0], tuple):  # (name, parameter) pairs: apply the group specs
            params = self.group_parameters(list(params))
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
                "scheduler_interval": self.scheduler_interval,
                "param_groups": [g.model_dump() for g in self.param_groups]}


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
            o, s = cfg.build([(f"{key}.{n}", p) for n, p in named] if cfg.param_groups else [p for _, p in named])
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
            if metrics is not None and c.scheduler_metric_adapter is not None:
                s.step(float(c.scheduler_metric_adapter(metrics)))
            elif metrics is not None and c.scheduler_metric in metrics:
                s.step(float(metrics[c.scheduler_metric]))
        else:
            s.step()


def step_lr_schedulers(scheds: list, configs: "list[OptimizerConfig] | None" = None, interval: str = "step",
                       metrics: dict | None = None) -> None:
    """Step learning-rate schedulers (the reference's name, ``training/optimizers.py:404-447``).  With their
    ``OptimizerConfig`` list only those of the given ``interval`` step, metric-driven ones with ``metrics``; without it
    every scheduler that is not metric-driven steps once."""
    if configs is not None:
        step_schedulers(scheds, configs, interval, metrics)
        return
    for s in scheds:
        if s is not None and not isinstance(s, torch.optim.lr_scheduler.ReduceLROnPlateau):
            s.step()
