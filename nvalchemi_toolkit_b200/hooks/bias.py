# SPDX-License-Identifier: Apache-2.0
"""``BiasedPotentialHook``: adds a user bias energy / force after the model evaluation
(reference ``nvalchemi/hooks/bias.py:40-173``)."""
from __future__ import annotations

from enum import Enum
from typing import Any, Callable


class BiasedPotentialHook:
    def __init__(self, bias_fn: Callable[[Any], tuple[Any, Any]], stage: Enum | None = None, frequency: int = 1,
                 inplace: bool = True) -> None:
        self.bias_fn, self.stage, self.frequency, self.inplace = bias_fn, stage, frequency, inplace

    def on_register(self, owner: Any) -> None:
        if self.stage is None:
            from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

            self.stage = DynamicsStage.AFTER_COMPUTE

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        e, f = self.bias_fn(b)
        if e is not None:
            e = e.reshape(b.energy.shape).to(b.energy.dtype)
            if self.inplace:
                b.energy.add_(e)
            else:
                b["energy"] = b.energy + e
        if f is not None:
            f = f.to(b.forces.dtype)
            if self.inplace:
                b.forces.add_(f)
            else:
                b["forces"] = b.forces + f
