# SPDX-License-Identifier: Apache-2.0
"""Small runtime helpers of the training loop (reference ``nvalchemi/training/runtime.py:36-230``)."""
from __future__ import annotations

import contextlib
import inspect
from typing import Any, Callable, Iterator

import torch


def move_to_devices(models: dict[str, torch.nn.Module], devices: list) -> dict[str, torch.nn.Module]:
    return {k: m.to(devices[min(i, len(devices) - 1)]) for i, (k, m) in enumerate(models.items())}


@contextlib.contextmanager
def freeze_unconfigured_models(models: dict[str, torch.nn.Module], optimizer_configs: dict) -> Iterator[None]:
    saved = []
    for k, m in models.items():
        if k not in optimizer_configs:
            for p in m.parameters():
                saved.append((p, p.requires_grad))
                p.requires_grad_(False)
    try:
        yield
    finally:
        for p, r in saved:
            p.requires_grad_(r)


@contextlib.contextmanager
def train_configured_models(models: dict[str, torch.nn.Module], optimizer_configs: dict) -> Iterator[None]:
    modes = {k: m.training for k, m in models.items()}
    for k, m in models.items():
        m.train(k in optimizer_configs)
    try:
        yield
    finally:
        for k, m in models.items():
            m.train(modes[k])


def configure_parallelism(strategy: str = "none", **kwargs: Any) -> None:
    """Only data parallelism through hooks is supported (as in the reference); other strategies are rejected."""
    if strategy != "none":
        raise NotImplementedError(f"parallelism strategy {strategy!r} is not supported; use DDPHook or "
                                  "FusedGradAllReduceHook for data parallel training")


def validate_training_fn(fn: Callable) -> None:
    params = list(inspect.signature(fn).parameters)
    if len(params) < 2:
        raise TypeError("training_fn must accept (model_or_models, batch)")
