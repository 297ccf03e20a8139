# SPDX-License-Identifier: Apache-2.0
"""Validation pass (reference ``nvalchemi/training/_validation.py:66-1012``): a context-managed loop that puts the models
in eval mode, accumulates every loss term in float64 weighted by the number of graphs, sums the accumulators over the
ranks and, on exit, restores what it touched: training modes AND parameter gradients (a validation pass between the
micro-batches of an accumulation window must not disturb the gradients collected so far).

``ValidationConfig`` carries the schedule (``every_n_steps`` / ``every_n_epochs``), the data (any re-iterable of batches:
a one-shot iterator would be empty from the second validation on and is rejected), an optional loss of its own (``loss_fn``;
default: the training loss at the current step and epoch, so weight schedules apply), ``enable_grad`` (conservative
models differentiate the energy for forces even in evaluation), per-batch callbacks (parity plots, error histograms)
and extra metrics computed from predictions and batch."""
from __future__ import annotations

from typing import Any, Callable, Iterable, Iterator, Mapping, Protocol

import torch
from pydantic import BaseModel, ConfigDict, field_validator, model_validator

from nvalchemi_toolkit_b200.training.distributed import all_reduce

Metric = Callable[[Any, Any], "torch.Tensor | float"]


class BatchValidationCallback(Protocol):
    """``ValidationConfig.batch_callback``: called once per validation batch with the batch, the model's predictions and
    the loss dictionary (parity plots, error histograms, outlier dumps)."""

    def __call__(self, batch: Any, predictions: dict, losses: dict) -> None: ...


def ensure_reiterable(value: Any) -> Any:
    """A generator / iterator can be consumed once; validation runs many times."""
    if value is None:
        return value
    if isinstance(value, Iterator):
        raise TypeError("validation data must be re-iterable (a list, DataLoader or Dataset-backed loader), not a one-shot "
                        f"iterator of type {type(value).__name__}")
    if not hasattr(value, "__iter__"):
        raise TypeError(f"validation data of type {type(value).__name__} is not iterable")
    return value


class ValidationConfig(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True)
    data: Any = None
    every_n_steps: int | None = None
    every_n_epochs: int | None = 1
    enable_grad: bool = True  # conservative models need autograd for forces even in evaluation
    loss_fn: Any = None       # default: the strategy's training loss
    metrics: dict[str, Metric] = {}
    batch_callback: Callable[[Any, dict, dict], None] | None = None
    max_batches: int | None = None
    use_inference_model: bool = True  # evaluate the strategy's inference model (EMA weights) when it has one

    @field_validator("data")
    @classmethod
    def _check_data(cls, v: Any) -> Any:
        return ensure_reiterable(v)

    @model_validator(mode="after")
    def _check_schedule(self) -> "ValidationConfig":
        for name in ("every_n_steps", "every_n_epochs", "max_batches"):
            value = getattr(self, name)
            if value is not None and value <= 0:
                raise ValueError(f"{name} must be positive or None, got {value}")
        return self


class _Accumulator:
    """Graph-weighted float64 sums of named scalars, reducible over ranks with one collective."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.sums: dict[str, torch.Tensor] = {}
        self.count = torch.zeros(1, dtype=torch.float64, device=device)
        self.batches = 0

    def update(self, scalars: Mapping[str, Any], weight: float) -> None:
        for k, v in scalars.items():
            t = v.detach().double().reshape(-1)[:1] if isinstance(v, torch.Tensor) else torch.tensor([float(v)], dtype=torch.float64)
            self.sums[k] = self.sums.get(k, torch.zeros(1, dtype=torch.float64, device=self.device)) + t.to(self.device) * weight
        self.count += weight
        self.batches += 1

    def summary(self, manager: Any) -> dict[str, float]:
        keys = sorted(self.sums)
        # ranks may hold different key sets only through a bug; the stacked layout assumes the same sorted keys everywhere
        stacked = torch.cat([self.sums[k] for k in keys] + [self.count])
        all_reduce(stacked, "sum", manager)
        total = float(stacked[-1].clamp_min(1))
        out = {k: float(stacked[i]) / total for i, k in enumerate(keys)}
        out["num_graphs"] = float(stacked[-1])
        return out


class ValidationLoop:
    def __init__(self, strategy: Any, model: Any, config: ValidationConfig | None) -> None:
        self.strategy, self.model, self.config = strategy, model, config or ValidationConfig()
        self._modes: list[tuple[torch.nn.Module, bool]] = []
        self._grads: list[tuple[torch.nn.Parameter, torch.Tensor | None]] = []

    @classmethod
    def from_training_strategy(cls, strategy: Any, config: ValidationConfig | None = None) -> "ValidationLoop":
        """The loop a strategy runs: its validation config and its inference model (EMA weights when a hook installed
        them), else the training model(s)."""
        cfg = config if config is not None else (strategy.validation_config or ValidationConfig())
        model = strategy.inference_model if (cfg.use_inference_model and strategy.inference_model is not None) else (
            strategy.models["main"] if strategy.single_model_input else strategy.models)
        return cls(strategy, model, cfg)

    def _modules(self) -> list[torch.nn.Module]:
        mods = list(self.model.values()) if isinstance(self.model, dict) else [self.model]
        seen: set[int] = set()
        return [m for m in mods if isinstance(m, torch.nn.Module) and not (id(m) in seen or seen.add(id(m)))]

    def __enter__(self) -> "ValidationLoop":
        for m in self._modules():
            self._modes.append((m, m.training))
            m.eval()
            for p in m.parameters():
                self._grads.append((p, p.grad))
                p.grad = None  # a stray backward inside a callback must not add to the training gradients
        return self

    def __exit__(self, *exc: Any) -> None:
        for p, g in self._grads:
            p.grad = g
        for m, was in self._modes:
            m.train(was)
        self._modes, self._grads = [], []

    def run(self, loader: Iterable) -> dict[str, Any]:
        s, cfg = self.strategy, self.config
        dev = s.devices[0]
        loss_fn = cfg.loss_fn if cfg.loss_fn is not None else s.loss_fn
        acc = _Accumulator(torch.device(dev))
        grad = torch.enable_grad() if cfg.enable_grad else torch.no_grad()
        with grad:
            for i, batch in enumerate(ensure_reiterable(loader)):
                if cfg.max_batches is not None and i >= cfg.max_batches:
                    break
                batch = batch.to(dev) if hasattr(batch, "to") else batch
                preds = s.training_fn(self.model, batch)
                losses = loss_fn(preds, batch, step=s.step_count, epoch=s.epoch_count)
                scalars = dict(losses)
                for name, fn in cfg.metrics.items():
                    scalars[f"metric/{name}"] = fn(preds, batch)
                acc.update(scalars, float(getattr(batch, "num_graphs", 1)))
                if cfg.batch_callback is not None:
                    cfg.batch_callback(batch, preds, losses)
        out: dict[str, Any] = acc.summary(s.distributed_manager) if acc.sums else {"num_graphs": 0.0}
        out["num_batches"] = acc.batches
        out["step"] = s.step_count
        out["epoch"] = s.epoch_count
        return out

    def execute(self, loader: Iterable | None = None) -> dict[str, Any]:
        """Enter, run over ``loader`` (default: the configured data), exit."""
        data = loader if loader is not None else self.config.data
        if data is None:
            raise ValueError("no validation data: pass a loader or set ValidationConfig.data")
        with self:
            return self.run(data)
