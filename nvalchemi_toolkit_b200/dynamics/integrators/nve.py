# SPDX-License-Identifier: Apache-2.0
"""Microcanonical velocity-Verlet integrator (reference ``nvalchemi/dynamics/integrators/nve.py:56-178``)."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import fs_to_internal_time
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics


class NVE(BaseDynamics):
    """``dt`` in femtoseconds (scalar or per-system tensor)."""

    #: the closing update is ``v += dt/2 F/m`` and nothing else: a domain decomposition may fuse it with its force return
    __dd_half_kick_finalize__ = True
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}

    def __init__(self, model: Any, dt: float | torch.Tensor, n_steps: int | None = None, hooks: list | None = None,
                 convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        self._dt_init = fs_to_internal_time(dt)

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        return {"dt": _ops._to_per_system(self._dt_init, n, template_batch.device, template_batch.positions.dtype)}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    def pre_update(self, batch: Batch) -> None:
        _ops.vv_position_update(batch.positions, batch.velocities, batch.forces, batch.atomic_masses,
                                self._state["dt"], batch.batch_idx)

    def post_update(self, batch: Batch) -> None:
        _ops.vv_velocity_finalize(batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"],
                                  batch.batch_idx)
