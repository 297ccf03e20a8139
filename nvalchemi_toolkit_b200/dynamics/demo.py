# SPDX-License-Identifier: Apache-2.0
"""Pure-torch velocity Verlet used in tests (reference ``nvalchemi/dynamics/demo.py:46-233``):
Euler fallback on the first step when no forces are known yet."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics


class DemoDynamics(BaseDynamics):
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"velocities", "positions"}

    def __init__(self, model: Any, n_steps: int, dt: float = 1.0, hooks: list | None = None,
                 convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, hooks=hooks, convergence_hook=convergence_hook, n_steps=n_steps, **kwargs)
        self.dt = dt
        self._prev_accelerations: torch.Tensor | None = None

    def pre_update(self, batch: Batch) -> None:
        forces = batch.forces
        masses = batch.atomic_masses.unsqueeze(-1)
        with torch.no_grad():
            if forces is not None and not torch.all(forces == 0):
                acc = forces / masses
                self._prev_accelerations = acc.clone()
                batch.positions.add_(batch.velocities * self.dt + 0.5 * acc * self.dt * self.dt)
            else:
                batch.positions.add_(batch.velocities * self.dt)

    def post_update(self, batch: Batch) -> None:
        with torch.no_grad():
            acc = batch.forces / batch.atomic_masses.unsqueeze(-1)
            prev = self._prev_accelerations
            if prev is not None and prev.shape == acc.shape:
                batch.velocities.add_(0.5 * (prev + acc) * self.dt)
            else:
                batch.velocities.add_(acc * self.dt)
