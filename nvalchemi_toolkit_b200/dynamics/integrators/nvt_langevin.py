# SPDX-License-Identifier: Apache-2.0
"""Langevin thermostat, BAOAB splitting (reference ``nvalchemi/dynamics/integrators/nvt_langevin.py:52-196``).

``dt`` in fs, ``temperature`` in K, ``friction`` in 1/fs.  The noise seed of step ``k`` is
``random_seed + k`` so a restarted trajectory reproduces the same noise."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import KB_EV, fs_to_internal_time, per_fs_to_internal_rate
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics


class NVTLangevin(BaseDynamics):
    #: the closing update is ``v += dt/2 F/m`` and nothing else: a domain decomposition may fuse it with its force return
    __dd_half_kick_finalize__ = True
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}
    __dd_thermo_kind__ = "local"

    def __init__(self, model: Any, dt: float | torch.Tensor, temperature: float | torch.Tensor,
                 friction: float | torch.Tensor, random_seed: int = 42, n_steps: int | None = None,
                 hooks: list | None = None, convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        self._dt_init = fs_to_internal_time(dt)
        self._temperature_init = temperature
        self._friction_init = per_fs_to_internal_rate(friction)
        self._random_seed = random_seed
        self.atom_ids: torch.Tensor | None = None  # global atom ids under domain decomposition

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        dev, dtype = template_batch.device, template_batch.positions.dtype
        return {"dt": _ops._to_per_system(self._dt_init, n, dev, dtype),
                "temperature": _ops._to_per_system(self._temperature_init, n, dev, dtype) * KB_EV,
                "friction": _ops._to_per_system(self._friction_init, n, dev, dtype)}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    def pre_update(self, batch: Batch) -> None:
        s = self._state
        _ops.langevin_half_step(batch.positions, batch.velocities, batch.forces, batch.atomic_masses, s["dt"],
                                s["temperature"], s["friction"], self._random_seed + self.step_count, batch.batch_idx,
                                self.atom_ids)

    def post_update(self, batch: Batch) -> None:
        _ops.langevin_finalize(batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"], batch.batch_idx)
