# SPDX-License-Identifier: Apache-2.0
"""Hook protocol, contexts and the registry mixin shared by dynamics and training.

Behavioural contract (reference ``nvalchemi/hooks/_protocol.py:27-89``,
``_context.py:31-139``, ``_registry.py:25-179``): a hook has ``frequency`` and
``stage``; it fires at its stage when ``step_count % frequency == 0``; a hook may
define ``_runs_on_stage(stage)`` to subscribe to several stages and
``on_register(owner)`` to react to registration; an engine may restrict the enum
type of accepted stages through ``_stage_type``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Mapping, Protocol, runtime_checkable

import torch


@runtime_checkable
class Hook(Protocol):
    frequency: int
    stage: Enum | None

    def __call__(self, ctx: "HookContext", stage: Enum) -> None: ...


@runtime_checkable
class CheckpointableHook(Protocol):
    def state_dict(self) -> Mapping[str, Any]: ...

    def load_state_dict(self, state: Mapping[str, Any]) -> None: ...


@dataclass(kw_only=True)
class HookContext:
    batch: Any
    model: Any = None
    global_rank: int = 0
    workflow: Any = None


@dataclass(kw_only=True)
class DynamicsContext(HookContext):
    step_count: int = 0
    converged_mask: torch.Tensor | None = None


@dataclass(kw_only=True)
class TrainContext(HookContext):
    step_count: int = 0
    global_step_count: int = 0
    batch_count: int = 0
    epoch_step_count: int = 0
    epoch: int = 0
    loss: torch.Tensor | None = None
    losses: dict[str, torch.Tensor] | None = None
    models: Any = None
    optimizers: list = field(default_factory=list)
    lr_schedulers: list = field(default_factory=list)
    gradients: dict[str, torch.Tensor] | None = None
    grad_scaler: Any = None
    validation: dict[str, Any] | None = None
    predictions: Any = None


def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


class HookRegistryMixin:
    """Flat hook list with stage/frequency dispatch."""

    hooks: list
    step_count: int
    _stage_type: Any = None

    def _init_hooks(self, hooks: list | None = None) -> None:
        self.hooks = []
        for h in hooks or ():
            self.register_hook(h)

    def register_hook(self, hook: Any, stage: Enum | None = None) -> None:
        freq = getattr(hook, "frequency", None)
        if not isinstance(freq, int) or isinstance(freq, bool) or freq < 1:
            raise ValueError(f"Hook frequency must be a positive integer, got {freq}")
        if stage is not None:
            hook.stage = stage
        on_register = getattr(hook, "on_register", None)
        if on_register is not None:
            if not callable(on_register):
                raise TypeError(f"Hook {type(hook).__name__}.on_register must be callable.")
            on_register(self)  # first: hooks that work for several engines pick their default stage here
        custom = getattr(hook, "_runs_on_stage", None) is not None
        if getattr(hook, "stage", None) is None and not custom:
            raise TypeError(
                f"Hook {type(hook).__name__} has no stage assigned. Pass stage= to the hook constructor "
                "or to register_hook()."
            )
        st = self._stage_type
        if st is not None and not custom and hook.stage is not None and not isinstance(hook.stage, st):
            names = st.__name__ if isinstance(st, type) else " | ".join(t.__name__ for t in st)
            raise TypeError(
                f"Hook {hook!r} has stage={hook.stage!r} (type {type(hook.stage).__name__}), but this engine "
                f"only accepts {names} stages."
            )
        self.hooks.append(hook)

    def _build_context(self, batch: Any) -> HookContext:
        return HookContext(batch=batch, model=getattr(self, "model", None), global_rank=_rank(), workflow=self)

    def _call_hooks(self, stage: Enum, batch: Any) -> None:
        if not self.hooks:
            return
        ctx = None
        for hook in self.hooks:
            runs = getattr(hook, "_runs_on_stage", None)
            if runs is not None:
                if not runs(stage):
                    continue
            elif stage != hook.stage:
                continue
            if self.step_count % hook.frequency == 0:
                if ctx is None:
                    ctx = self._build_context(batch)
                hook(ctx, stage)

    def _open_hooks(self) -> None:
        for h in self.hooks:
            fn = getattr(h, "__enter__", None)
            if fn is not None:
                fn()

    def _close_hooks(self) -> None:
        for h in self.hooks:
            fn = getattr(h, "__exit__", None)
            if fn is not None:
                fn(None, None, None)
