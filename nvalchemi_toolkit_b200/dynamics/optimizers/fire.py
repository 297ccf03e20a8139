# SPDX-License-Identifier: Apache-2.0
"""FIRE structure relaxation (reference ``nvalchemi/dynamics/optimizers/fire.py:69-539``).

The whole iteration runs in ``pre_update`` on the forces of the previous evaluation; ``post_update``
is empty.  Defaults: ``maxstep 0.2, n_min 5, f_dec 0.5, f_inc 1.1, alpha_start 0.1, f_alpha 0.99``,
``dt_max = 10 dt``, ``dt_min = 0.02 dt``.  ``dt`` is in internal time units (as in the reference)."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics

_FIRE_DEFAULTS = {"maxstep": 0.2, "n_min": 5, "f_dec": 0.5, "f_inc": 1.1, "alpha_start": 0.1, "f_alpha": 0.99}


class FIRE(BaseDynamics):
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}
    __dd_thermo_kind__ = "fire"

    def __init__(self, model: Any, dt: float | torch.Tensor, dt_max: float | torch.Tensor | None = None,
                 dt_min: float | torch.Tensor | None = None, maxstep: float = 0.2, n_min: int = 5, f_dec: float = 0.5,
                 f_inc: float = 1.1, alpha_start: float = 0.1, f_alpha: float = 0.99, uphill: bool | torch.Tensor = False,
                 n_steps: int | None = None, hooks: list | None = None, convergence_hook: Any = None,
                 **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        self._dt_init, self._dt_max_init, self._dt_min_init = dt, dt_max, dt_min
        self.maxstep, self.n_min, self.f_dec, self.f_inc = maxstep, n_min, f_dec, f_inc
        self.alpha_start, self.f_alpha = alpha_start, f_alpha
        self._uphill_init = uphill
        self.compute_reductions = True  # a domain-decomposition coordinator supplies global sums instead
        self.reduce_max = None          # ... and the cross-rank maximum for the step-length cap

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        dev, dtype = template_batch.device, template_batch.positions.dtype
        dt = _ops._to_per_system(self._dt_init, n, dev, dtype)
        full = lambda v, dt_=dtype: torch.full((n,), v, dtype=dt_, device=dev)  # noqa: E731
        up = self._uphill_init
        uphill = up.expand(n).to(torch.int32).to(dev).contiguous() if isinstance(up, torch.Tensor) \
            else full(1 if up else 0, torch.int32)
        return {
            "dt": dt,
            "dt_max": _ops._to_per_system(self._dt_max_init, n, dev, dtype) if self._dt_max_init is not None else dt * 10.0,
            "dt_min": _ops._to_per_system(self._dt_min_init, n, dev, dtype) if self._dt_min_init is not None else dt * 0.02,
            "alpha": full(self.alpha_start), "alpha_start": full(self.alpha_start), "f_alpha": full(self.f_alpha),
            "maxstep": full(self.maxstep), "n_min": full(self.n_min, torch.int32), "f_dec": full(self.f_dec),
            "f_inc": full(self.f_inc), "uphill_flag": uphill, "n_steps_positive": full(0, torch.int32),
            "vf": full(0.0), "vv": full(0.0), "ff": full(0.0),
        }

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    def pre_update(self, batch: Batch) -> None:
        s = self._state
        _ops.fire_step(batch.positions, batch.velocities, batch.forces, batch.atomic_masses, s["alpha"], s["dt"],
                       s["n_steps_positive"], s["alpha_start"], s["f_alpha"], s["dt_min"], s["dt_max"], s["maxstep"],
                       s["n_min"], s["f_dec"], s["f_inc"], s["uphill_flag"], vf=s["vf"], vv=s["vv"], ff=s["ff"],
                       batch_idx=batch.batch_idx, compute_reductions=self.compute_reductions, reduce_max=self.reduce_max)

    def post_update(self, batch: Batch) -> None:
        pass
