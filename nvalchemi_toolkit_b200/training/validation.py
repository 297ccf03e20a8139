# SPDX-License-Identifier: Apache-2.0
"""Validation pass (reference ``nvalchemi/training/_validation.py:66-1012``): context-managed loop that puts the models
in eval mode, accumulates loss terms in fp64 weighted by the number of graphs, sums the accumulators over ranks and
restores the training mode on exit."""
from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
from pydantic import BaseModel, ConfigDict

from nvalchemi_toolkit_b200.training.distributed import all_reduce


class ValidationConfig(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True)
    data: Any = None
    every_n_steps: int | None = None
    every_n_epochs: int | None = 1
    enable_grad: bool = True  # conservative models need autograd for forces even in evaluation
    batch_callback: Callable[[Any, dict, dict], None] | None = None
    max_batches: int | None = None


class ValidationLoop:
    def __init__(self, strategy: Any, model: Any, config: ValidationConfig | None) -> None:
        self.strategy, self.model, self.config = strategy, model, config or ValidationConfig()
        self._modes: list[tuple[torch.nn.Module, bool]] = []

    def __enter__(self) -> "ValidationLoop":
        mods = self.model.values() if isinstance(self.model, dict) else [self.model]
        for m in mods:
            self._modes.append((m, m.training))
            m.eval()
        return self

    def __exit__(self, *exc: Any) -> None:
        for m, was in self._modes:
            m.train(was)

    def run(self, loader: Iterable) -> dict[str, Any]:
        s = self.strategy
        dev = s.devices[0]
        sums: dict[str, torch.Tensor] = {}
        count = torch.zeros(1, dtype=torch.float64, device=dev)
        grad = torch.enable_grad() if self.config.enable_grad else torch.no_grad()
        with grad:
            for i, batch in enumerate(loader):
                if self.config.max_batches is not None and i >= self.config.max_batches:
                    break
                batch = batch.to(dev) if hasattr(batch, "to") else batch
                preds = s.training_fn(self.model, batch)
                losses = s.loss_fn(preds, batch, step=s.step_count, epoch=s.epoch_count)
                n = float(getattr(batch, "num_graphs", 1))
                for k, v in losses.items():
                    sums[k] = sums.get(k, torch.zeros(1, dtype=torch.float64, device=dev)) + v.detach().double() * n
                count += n
                if self.config.batch_callback is not None:
                    self.config.batch_callback(batch, preds, losses)
        keys = sorted(sums)
        if keys:
            stacked = torch.cat([sums[k] for k in keys] + [count])
            all_reduce(stacked, "sum", s.distributed_manager)
            total = float(stacked[-1].clamp_min(1))
            out = {k: float(stacked[i]) / total for i, k in enumerate(keys)}
        else:
            out = {}
        out["num_graphs"] = float(count)
        out["step"] = s.step_count
        return out
