# SPDX-License-Identifier: Apache-2.0
"""Isothermal-isobaric (NPT) and isoenthalpic (NPH) dynamics, Martyna-Tobias-Klein equations.

Reference: ``nvalchemi/dynamics/integrators/npt.py`` / ``nph.py`` and the ``npt_*`` / ``nph_*`` ops
(``dynamics/_ops/npt_nph.py:59-911``).  The cell strain rate is a 3 x 3 matrix ``v_g`` per system: a multiple of the identity
(``isotropic``), diagonal (``anisotropic``) or a full symmetric matrix (``triclinic``: shear components of the pressure
tensor drive the cell angles; the symmetric form keeps the cell from rotating).  Particle velocities and positions are
advanced with the matrix exponentials of ``v_g`` (one fused per-atom kernel each, ``_ops.affine_rows_``).  Particles and
barostat carry separate Nose-Hoover chains in NPT; NPH drops both chains.  The model must provide ``stress`` (tensile
positive).  Pressure is given in eV/A^3."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import KB_EV, fs_to_internal_time
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics
from nvalchemi_toolkit_b200.dynamics.integrators.nvt_nose_hoover import nhc_chain_update, nhc_compute_masses


def compute_kinetic_tensor(velocities: torch.Tensor, masses: torch.Tensor, batch_idx: torch.Tensor, m: int) -> torch.Tensor:
    """``sum_i m_i v_i (x) v_i`` per system, ``[M,3,3]``."""
    return _ops.compute_kinetic_tensor(velocities, masses, batch_idx, m)


compute_pressure_tensor = _ops.compute_pressure_tensor


class NPT(BaseDynamics):
    __needs_keys__ = {"forces", "stress"}
    __provides_keys__ = {"positions", "velocities", "cell"}
    __dd_thermo_kind__ = "npt"
    _thermostat = True

    def __init__(self, model: Any, dt: float, temperature: float, pressure: float, barostat_time: float,
                 thermostat_time: float, pressure_coupling: str = "isotropic", chain_length: int = 3,
                 n_steps: int | None = None, hooks: list | None = None, convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        if pressure_coupling not in ("isotropic", "anisotropic", "triclinic"):
            raise ValueError("pressure_coupling must be 'isotropic', 'anisotropic' or 'triclinic'")
        self._dt_init = fs_to_internal_time(dt)
        self._temperature_init, self._pressure_init = temperature, pressure
        self._tau_b, self._tau_t = fs_to_internal_time(barostat_time), fs_to_internal_time(thermostat_time)
        self.pressure_coupling, self.chain_length = pressure_coupling, chain_length
        self.ke_reduce = None     # cross-rank sums installed by a domain-decomposition coordinator
        self.count_reduce = None
        if "stress" not in model.model_config.active_outputs:
            model.model_config.active_outputs = set(model.model_config.active_outputs) | {"stress"}

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        dev, dtype = template_batch.device, template_batch.positions.dtype
        z = torch.zeros(n, self.chain_length, dtype=dtype, device=dev)
        return {"dt": _ops._to_per_system(self._dt_init, n, dev, dtype),
                "kT": _ops._to_per_system(self._temperature_init, n, dev, dtype) * KB_EV,
                "p_ext": _ops._to_per_system(self._pressure_init, n, dev, dtype),
                "tau_t": _ops._to_per_system(self._tau_t, n, dev, dtype),
                "tau_b": _ops._to_per_system(self._tau_b, n, dev, dtype),
                "eta": z.clone(), "eta_dot": z.clone(), "xi": z.clone(), "xi_dot": z.clone(),
                "v_g": torch.zeros(n, 3, 3, dtype=dtype, device=dev)}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    # -- pieces ------------------------------------------------------------------
    def _ndof(self, batch: Batch) -> torch.Tensor:
        n = 3.0 * batch.num_nodes_per_graph.to(batch.positions.dtype)
        return n if self.count_reduce is None else self.count_reduce(n)

    def _barostat_mass(self, batch: Batch) -> torch.Tensor:
        s = self._state
        return _ops.compute_barostat_mass(self._ndof(batch), s["kT"], s["tau_b"])

    def _project(self, g: torch.Tensor) -> torch.Tensor:
        """Restrict a 3 x 3 generalised force to the degrees of freedom of the coupling mode."""
        return _ops.project_cell_force(g, self.pressure_coupling)

    def _thermostat_half(self, batch: Batch) -> None:
        if not self._thermostat:
            return
        _ops.npt_thermostat_half_step(batch.velocities, batch.atomic_masses, batch.batch_idx, self._state["v_g"], self._state,
                                      self._ndof(batch), self._barostat_mass(batch), self.pressure_coupling,
                                      self.chain_length, ke_reduce=self.ke_reduce)

    def _barostat_half(self, batch: Batch) -> None:
        s, m = self._state, batch.num_graphs
        vol = torch.linalg.det(batch.cell.reshape(m, 3, 3)).abs()
        K = compute_kinetic_tensor(batch.velocities, batch.atomic_masses, batch.batch_idx, m)
        if self.ke_reduce is not None:
            K = self.ke_reduce(K)
        stress = getattr(batch, "stress", None)
        stress = torch.zeros_like(K) if stress is None else stress.reshape(m, 3, 3)
        P = compute_pressure_tensor(K, stress, vol)
        ke2 = torch.diagonal(K, dim1=1, dim2=2).sum(-1)
        _ops.npt_barostat_half_step(s["v_g"], P, s["p_ext"], vol, ke2, self._ndof(batch), self._barostat_mass(batch), s["dt"],
                                    self.pressure_coupling)

    def _damping(self, batch: Batch) -> torch.Tensor:
        """``exp(-dt/2 (v_g + tr(v_g) / N_f))`` per system."""
        return _ops.npt_cell_damping(self._state["v_g"], self._ndof(batch), self._state["dt"])

    def _velocity_half(self, batch: Batch) -> None:
        """Damp by the cell motion, then half kick (one fused per-atom kernel)."""
        s = self._state
        _ops.npt_velocity_half_step(batch.velocities, batch.forces, batch.atomic_masses, s["v_g"], self._ndof(batch), s["dt"],
                                    batch.batch_idx, kick_first=False)

    def _velocity_half_reverse(self, batch: Batch) -> None:
        """Half kick, then damp (the mirror image of :meth:`_velocity_half`)."""
        s = self._state
        _ops.npt_velocity_half_step(batch.velocities, batch.forces, batch.atomic_masses, s["v_g"], self._ndof(batch), s["dt"],
                                    batch.batch_idx, kick_first=True)

    def _drift(self, batch: Batch) -> None:
        """``r <- r exp(dt v_g) + dt v exp(dt v_g / 2)``; the lattice vectors (cell rows) follow ``exp(dt v_g)``."""
        s = self._state
        grow = _ops.npt_position_update(batch.positions, batch.velocities, s["v_g"], s["dt"], batch.batch_idx)
        _ops.npt_cell_update(batch.cell, grow)

    # -- step ------------------------------------------------------------------------
    def pre_update(self, batch: Batch) -> None:
        self._thermostat_half(batch)
        self._barostat_half(batch)
        self._velocity_half_reverse(batch)
        self._drift(batch)

    def post_update(self, batch: Batch) -> None:
        self._velocity_half(batch)
        self._barostat_half(batch)
        self._thermostat_half(batch)


def __getattr__(name: str) -> Any:
    """``NPH`` lives in :mod:`nvalchemi_toolkit_b200.dynamics.integrators.nph`; importing it from here still works."""
    if name == "NPH":
        from nvalchemi_toolkit_b200.dynamics.integrators.nph import NPH

        return NPH
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
