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


def configure_dataloader(dataset: Any, *, batch_size: int, shuffle: bool | None = None, sampler: Any = None,
                         batch_sampler: Any = None, **loader_kwargs: Any) -> Any:
    """The package's :class:`~nvalchemi_toolkit_b200.data.datapipes.DataLoader` with the defaulting rules of the
    reference helper (``training/runtime.py:154-202``): ``shuffle`` defaults to ``True`` unless an order is given
    (``sampler`` / ``batch_sampler``); asking for both shuffling and an explicit order is an error.  A ``sampler`` (an
    iterable of indices with ``__len__`` and optionally ``set_epoch``) is cut into batches of ``batch_size``."""
    from nvalchemi_toolkit_b200.data.datapipes import DataLoader

    ordered = sampler is not None or batch_sampler is not None
    if shuffle is True and ordered:
        raise ValueError("shuffle=True is incompatible with sampler / batch_sampler: the sampler decides the order")
    if sampler is not None and batch_sampler is not None:
        raise ValueError("give a sampler or a batch_sampler, not both")
    if sampler is not None:
        batch_sampler = _BatchesOf(sampler, batch_size, bool(loader_kwargs.get("drop_last", False)))
    return DataLoader(dataset, batch_size=batch_size, shuffle=(not ordered) if shuffle is None else shuffle,
                      batch_sampler=batch_sampler, **loader_kwargs)


class _BatchesOf:
    """Index sampler -> batch sampler."""

    def __init__(self, sampler: Any, batch_size: int, drop_last: bool) -> None:
        self.sampler, self.batch_size, self.drop_last = sampler, int(batch_size), drop_last

    def set_epoch(self, epoch: int) -> None:
        if hasattr(self.sampler, "set_epoch"):
            self.sampler.set_epoch(epoch)

    def __iter__(self) -> Iterator[list[int]]:
        buf: list[int] = []
        for i in self.sampler:
            buf.append(int(i))
            if len(buf) == self.batch_size:
                yield buf
                buf = []
        if buf and not self.drop_last:
            yield buf

    def __len__(self) -> int:
        n = len(self.sampler)
        return n // self.batch_size if self.drop_last else -(-n // self.batch_size)
