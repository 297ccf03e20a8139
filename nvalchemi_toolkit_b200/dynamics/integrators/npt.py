# SPDX-License-Identifier: Apache-2.0
"""Isothermal-isobaric (NPT) and isoenthalpic (NPH) dynamics, Martyna-Tobias-Klein equations.

Reference: ``nvalchemi/dynamics/integrators/npt.py`` / ``nph.py`` and the ``npt_*`` / ``nph_*`` ops
(``dynamics/_ops/npt_nph.py:59-911``).  The cell has one strain-rate degree of freedom per system (``isotropic``) or one
per axis (``anisotropic``); ``triclinic`` is accepted and treated per axis after cell alignment.  Particles and barostat
carry separate Nose-Hoover chains in NPT; NPH drops both chains.  The model must provide ``stress`` (tensile positive).
Pressure is given in eV/A^3."""
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
    kt = (masses[:, None, None] * velocities[:, :, None] * velocities[:, None, :]).reshape(-1, 9)
    return _ops.segmented_sum(kt, batch_idx, m).reshape(m, 3, 3)


def compute_pressure_tensor(kinetic_tensor: torch.Tensor, stress: torch.Tensor, volume: torch.Tensor) -> torch.Tensor:
    """``P = K / V - sigma`` (``sigma`` tensile positive)."""
    return kinetic_tensor / volume[:, None, None] - stress


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
                "v_eps": torch.zeros(n, 3, dtype=dtype, device=dev)}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    # -- pieces ------------------------------------------------------------------
    def _ndof(self, batch: Batch) -> torch.Tensor:
        n = 3.0 * batch.num_nodes_per_graph.to(batch.positions.dtype)
        return n if self.count_reduce is None else self.count_reduce(n)

    def _barostat_mass(self, batch: Batch) -> torch.Tensor:
        s = self._state
        return (self._ndof(batch) + 3.0) * s["kT"] * s["tau_b"] ** 2

    def _thermostat_half(self, batch: Batch) -> None:
        if not self._thermostat:
            return
        s, m = self._state, batch.num_graphs
        ndof = self._ndof(batch)
        ke2 = 2.0 * _ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, m)
        if self.ke_reduce is not None:
            ke2 = self.ke_reduce(ke2)
        Q = nhc_compute_masses(ndof, s["kT"], s["tau_t"], self.chain_length)
        scale = nhc_chain_update(ke2, s["eta"], s["eta_dot"], Q, s["kT"], ndof, s["dt"])
        _ops.velocity_rescale(batch.velocities, scale, batch.batch_idx)
        W = self._barostat_mass(batch)
        nb = torch.full_like(ndof, 1.0 if self.pressure_coupling == "isotropic" else 3.0)
        kb2 = W * (s["v_eps"] ** 2).sum(-1) * (1.0 if self.pressure_coupling != "isotropic" else 1.0 / 3.0)
        Qb = nhc_compute_masses(nb, s["kT"], s["tau_b"], self.chain_length)
        sb = nhc_chain_update(kb2, s["xi"], s["xi_dot"], Qb, s["kT"], nb, s["dt"])
        s["v_eps"].mul_(sb.unsqueeze(-1))

    def _barostat_half(self, batch: Batch) -> None:
        s, m = self._state, batch.num_graphs
        cell = batch.cell.reshape(m, 3, 3)
        vol = torch.linalg.det(cell).abs()
        K = compute_kinetic_tensor(batch.velocities, batch.atomic_masses, batch.batch_idx, m)
        if self.ke_reduce is not None:
            K = self.ke_reduce(K)
        stress = getattr(batch, "stress", None)
        stress = torch.zeros_like(K) if stress is None else stress.reshape(m, 3, 3)
        P = compute_pressure_tensor(K, stress, vol)
        ke2 = torch.diagonal(K, dim1=1, dim2=2).sum(-1)
        ndof = self._ndof(batch)
        W = self._barostat_mass(batch)
        pdiag = torch.diagonal(P, dim1=1, dim2=2)
        if self.pressure_coupling == "isotropic":
            pdiag = pdiag.mean(-1, keepdim=True).expand(m, 3)
        g = (vol.unsqueeze(-1) * (pdiag - s["p_ext"].unsqueeze(-1)) + (ke2 / ndof).unsqueeze(-1)) / W.unsqueeze(-1)
        s["v_eps"].add_(0.5 * s["dt"].unsqueeze(-1) * g)

    def _velocity_half(self, batch: Batch) -> None:
        s = self._state
        b = batch.batch_idx.long()
        ndof = self._ndof(batch)
        alpha = 1.0 + 3.0 / ndof
        tr = s["v_eps"].sum(-1) / 3.0
        damp = torch.exp(-0.5 * s["dt"].unsqueeze(-1) * (s["v_eps"] + ((alpha - 1.0) * tr).unsqueeze(-1)))
        batch.velocities.mul_(damp[b])
        _ops.vv_velocity_finalize(batch.velocities, batch.forces, batch.atomic_masses, s["dt"], batch.batch_idx)

    def _velocity_half_reverse(self, batch: Batch) -> None:
        s = self._state
        b = batch.batch_idx.long()
        ndof = self._ndof(batch)
        alpha = 1.0 + 3.0 / ndof
        tr = s["v_eps"].sum(-1) / 3.0
        _ops.vv_velocity_finalize(batch.velocities, batch.forces, batch.atomic_masses, s["dt"], batch.batch_idx)
        damp = torch.exp(-0.5 * s["dt"].unsqueeze(-1) * (s["v_eps"] + ((alpha - 1.0) * tr).unsqueeze(-1)))
        batch.velocities.mul_(damp[b])

    def _drift(self, batch: Batch) -> None:
        s, m = self._state, batch.num_graphs
        b = batch.batch_idx.long()
        dt = s["dt"].unsqueeze(-1)
        grow = torch.exp(dt * s["v_eps"])
        half = torch.exp(0.5 * dt * s["v_eps"])
        batch.positions.mul_(grow[b]).add_(batch.velocities * (dt * half)[b])
        cell = batch.cell.reshape(m, 3, 3)
        cell.mul_(grow.unsqueeze(1))  # column d of every lattice vector scales with axis d

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


class NPH(NPT):
    __dd_thermo_kind__ = "nph"
    _thermostat = False

    def __init__(self, model: Any, dt: float, pressure: float, barostat_time: float,
                 pressure_coupling: str = "isotropic", temperature: float = 300.0, n_steps: int | None = None,
                 hooks: list | None = None, convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, dt=dt, temperature=temperature, pressure=pressure, barostat_time=barostat_time,
                         thermostat_time=barostat_time, pressure_coupling=pressure_coupling, n_steps=n_steps, hooks=hooks,
                         convergence_hook=convergence_hook, **kwargs)
