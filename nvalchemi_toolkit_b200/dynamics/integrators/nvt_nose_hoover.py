# SPDX-License-Identifier: Apache-2.0
"""Nose-Hoover-chain thermostat (MTK equations, Yoshida-Suzuki factorisation).

Reference: ``nvalchemi/dynamics/integrators/nvt_nose_hoover.py`` and the ``nhc_*`` ops
(``dynamics/_ops/nose_hoover.py:42-325``).  Per-system chain state ``eta, eta_dot [M, C]`` lives in ``_state`` and
follows the systems through inflight refills.  Chain masses ``Q_1 = N_f kT tau^2``, ``Q_k = kT tau^2``."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import KB_EV, fs_to_internal_time
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics

_YS = _ops._YS_W
nhc_compute_masses = _ops.nhc_compute_masses


def nhc_chain_update(ke2: torch.Tensor, eta: torch.Tensor, eta_dot: torch.Tensor, Q: torch.Tensor, kT: torch.Tensor,
                     ndof: torch.Tensor, dt: torch.Tensor, yoshida_order: int = 3) -> torch.Tensor:
    """Half-step propagation of the chains.  ``ke2 = 2 KE`` per system (updated in place); returns the velocity scale."""
    return _ops.nhc_chain_scalar(ke2, eta, eta_dot, Q, kT, ndof, dt, yoshida_order)


class NVTNoseHoover(BaseDynamics):
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}
    __dd_thermo_kind__ = "nhc"

    def __init__(self, model: Any, dt: float | torch.Tensor, temperature: float | torch.Tensor,
                 thermostat_time: float | torch.Tensor, chain_length: int = 3, yoshida_order: int = 3,
                 n_steps: int | None = None, hooks: list | None = None, convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        if yoshida_order not in _YS:
            raise ValueError("yoshida_order must be 1, 3 or 5")
        self._dt_init = fs_to_internal_time(dt)
        self._temperature_init = temperature
        self._tau_init = fs_to_internal_time(thermostat_time)
        self.chain_length, self.yoshida_order = chain_length, yoshida_order
        self.ke_reduce = None  # a domain-decomposition coordinator may install a cross-rank sum here
        self.count_reduce = None  # ... and the cross-rank atom count (degrees of freedom)

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        dev, dtype = template_batch.device, template_batch.positions.dtype
        z = torch.zeros(n, self.chain_length, dtype=dtype, device=dev)
        return {"dt": _ops._to_per_system(self._dt_init, n, dev, dtype),
                "kT": _ops._to_per_system(self._temperature_init, n, dev, dtype) * KB_EV,
                "tau": _ops._to_per_system(self._tau_init, n, dev, dtype), "eta": z.clone(), "eta_dot": z.clone()}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    def _thermostat_half(self, batch: Batch) -> None:
        s = self._state
        m = batch.num_graphs
        ke2 = 2.0 * _ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, m)
        if self.ke_reduce is not None:
            ke2 = self.ke_reduce(ke2)
        ndof = 3.0 * batch.num_nodes_per_graph.to(ke2.dtype)
        if self.count_reduce is not None:
            ndof = self.count_reduce(ndof)
        Q = nhc_compute_masses(ndof, s["kT"], s["tau"], self.chain_length)
        scale = nhc_chain_update(ke2, s["eta"], s["eta_dot"], Q, s["kT"], ndof, s["dt"], self.yoshida_order)
        _ops.velocity_rescale(batch.velocities, scale, batch.batch_idx)

    def pre_update(self, batch: Batch) -> None:
        self._thermostat_half(batch)
        _ops.vv_position_update(batch.positions, batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"],
                                batch.batch_idx)

    def post_update(self, batch: Batch) -> None:
        _ops.vv_velocity_finalize(batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"], batch.batch_idx)
        self._thermostat_half(batch)
