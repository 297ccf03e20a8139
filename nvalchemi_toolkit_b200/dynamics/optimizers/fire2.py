# SPDX-License-Identifier: Apache-2.0
"""FIRE2 relaxation (Guenole et al. 2020) with optional cell degrees of freedom.

Reference: ``nvalchemi/dynamics/optimizers/fire2.py:62-372`` (defaults ``delaystep 60, dtgrow 1.05, dtshrink 0.75,
alphashrink 0.985, alpha0 0.09, tmax 0.08, tmin 0.005, maxstep 0.1``).  Per system: ``P = F.v``; ``P > 0`` for more than
``delaystep`` steps grows ``dt`` and shrinks ``alpha``; ``P <= 0`` shrinks ``dt``, resets ``alpha``, steps back half a
step and zeroes the velocity; then a semi-implicit Euler step with velocity mixing and a per-system step cap."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics
from nvalchemi_toolkit_b200.ops import _native


def fire2_step_coord(positions, velocities, forces, batch_idx, alpha, dt, nsteps_inc, *, delaystep, dtgrow, dtshrink,
                     alphashrink, alpha0, tmax, tmin, maxstep, reduce=None, reduce_max=None) -> None:
    m = alpha.shape[0]
    if (_native.available() and hasattr(torch.ops.nvalchemi, "fire2_step") and positions.is_contiguous()
            and velocities.is_contiguous() and forces.is_contiguous() and alpha.dtype == positions.dtype == dt.dtype
            and nsteps_inc.dtype == torch.int32):
        # four kernel phases; a domain decomposition reduces the per-system sums between them
        op = torch.ops.nvalchemi.fire2_step
        sums = torch.empty(m, 3, dtype=torch.float64, device=positions.device)
        max_dr = torch.empty(m, dtype=torch.float32, device=positions.device)
        args = (positions, velocities, forces, batch_idx.to(torch.int32), alpha, dt, nsteps_inc, sums, max_dr, int(delaystep),
                float(dtgrow), float(dtshrink), float(alphashrink), float(alpha0), float(tmax), float(tmin), float(maxstep))
        if reduce is None and reduce_max is None:
            op(*args, 0)
            return
        op(*args, 1)
        if reduce is not None:
            sums[:, 0] = reduce(sums[:, 0].contiguous())
        op(*args, 2)
        if reduce is not None:
            sums[:, 1], sums[:, 2] = reduce(sums[:, 1].contiguous()), reduce(sums[:, 2].contiguous())
        op(*args, 3)
        if reduce_max is not None:
            max_dr.copy_(reduce_max(max_dr))
        op(*args, 4)
        return
    b = batch_idx.long()
    z = torch.zeros(m, dtype=torch.float64, device=positions.device)
    vf = z.clone().index_add_(0, b, (velocities.double() * forces.double()).sum(-1))
    if reduce is not None:
        vf = reduce(vf)
    pos_p = (vf > 0).to(positions.dtype)
    neg = vf <= 0
    nsteps_inc.copy_(torch.where(neg, torch.zeros_like(nsteps_inc), nsteps_inc + 1))
    grow = (~neg) & (nsteps_inc > delaystep)
    dt.copy_(torch.where(grow, torch.clamp(dt * dtgrow, max=tmax), torch.where(neg, torch.clamp(dt * dtshrink, min=tmin), dt)))
    alpha.copy_(torch.where(grow, alpha * alphashrink, torch.where(neg, torch.full_like(alpha, alpha0), alpha)))
    h = dt[b].unsqueeze(-1)
    # uphill: step back half a step and stop
    positions.sub_(0.5 * h * velocities * neg[b].unsqueeze(-1).to(positions.dtype))
    velocities.mul_(pos_p[b].unsqueeze(-1))
    velocities.add_(h * forces)
    vv = z.clone().index_add_(0, b, (velocities.double() ** 2).sum(-1))
    ff = z.clone().index_add_(0, b, (forces.double() ** 2).sum(-1))
    if reduce is not None:
        vv, ff = reduce(vv), reduce(ff)
    mix = (alpha * torch.sqrt(vv / ff.clamp_min(1e-300)).to(alpha.dtype))[b].unsqueeze(-1)
    velocities.mul_((1.0 - alpha)[b].unsqueeze(-1)).add_(mix * forces)
    dr = h * velocities
    mx = torch.zeros(m, dtype=dr.dtype, device=dr.device).scatter_reduce(0, b, dr.norm(dim=-1), "amax", include_self=True)
    if reduce_max is not None:
        mx = reduce_max(mx)
    scale = torch.where(mx > maxstep, maxstep / mx.clamp_min(1e-30), torch.ones_like(mx))
    positions.add_(scale[b].unsqueeze(-1) * dr)


class FIRE2(BaseDynamics):
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}
    __dd_thermo_kind__ = "fire"

    def __init__(self, model: Any, dt: float = 0.01, delaystep: int = 60, dtgrow: float = 1.05, dtshrink: float = 0.75,
                 alphashrink: float = 0.985, alpha0: float = 0.09, tmax: float = 0.08, tmin: float = 0.005,
                 maxstep: float = 0.1, n_steps: int | None = None, hooks: list | None = None,
                 convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, n_steps=n_steps, hooks=hooks, convergence_hook=convergence_hook, **kwargs)
        self._dt_init = dt
        self.hp = dict(delaystep=delaystep, dtgrow=dtgrow, dtshrink=dtshrink, alphashrink=alphashrink, alpha0=alpha0,
                       tmax=tmax, tmin=tmin, maxstep=maxstep)
        self.reduce = None      # cross-rank sum installed by a domain-decomposition coordinator
        self.reduce_max = None  # cross-rank maximum (step-length limiter)

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        dev, dtype = template_batch.device, template_batch.positions.dtype
        return {"dt": _ops._to_per_system(self._dt_init, n, dev, dtype),
                "alpha": torch.full((n,), self.hp["alpha0"], dtype=dtype, device=dev),
                "nsteps_inc": torch.zeros(n, dtype=torch.int32, device=dev)}

    def _init_state(self, batch: Batch) -> None:
        self._state = self._make_new_state(batch.num_graphs, batch)

    def pre_update(self, batch: Batch) -> None:
        s = self._state
        fire2_step_coord(batch.positions, batch.velocities, batch.forces, batch.batch_idx, s["alpha"], s["dt"],
                         s["nsteps_inc"], reduce=self.reduce, reduce_max=self.reduce_max, **self.hp)

    def post_update(self, batch: Batch) -> None:
        pass


class _CellFilterMixin:
    """Extends a position optimiser with cell degrees of freedom driven by the stress (unit-cell filter):
    generalised coordinates = (positions, cell rows), generalised forces = (forces, -V sigma applied to the cell)."""

    cell_factor: float | None = None

    def _cell_step(self, batch: Batch, step_fn: Any) -> None:
        m = batch.num_graphs
        cell = batch.cell.reshape(m, 3, 3)
        stress = batch.stress.reshape(m, 3, 3)
        n_at = batch.num_nodes_per_graph.to(cell.dtype)
        factor = n_at if self.cell_factor is None else torch.full_like(n_at, self.cell_factor)
        cell_force = _ops.stress_to_cell_force(cell, stress, factor)
        frac = torch.einsum("ni,nij->nj", batch.positions, torch.linalg.inv(cell)[batch.batch_idx.long()])
        old_cell = cell.clone()
        step_fn(cell_force)
        new_cell = batch.cell.reshape(m, 3, 3)
        # atoms follow the cell deformation (fractional coordinates of the position update are kept)
        delta = torch.einsum("ni,nij->nj", frac, (new_cell - old_cell)[batch.batch_idx.long()])
        batch.positions.add_(delta)


class FIRE2VariableCell(FIRE2, _CellFilterMixin):
    __needs_keys__ = {"forces", "stress"}
    __provides_keys__ = {"positions", "velocities", "cell"}

    def __init__(self, model: Any, *a: Any, cell_factor: float | None = None, **k: Any) -> None:
        super().__init__(model, *a, **k)
        self.cell_factor = cell_factor
        model.model_config.active_outputs = set(model.model_config.active_outputs) | {"stress"}

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        st = super()._make_new_state(n, template_batch)
        st["cell_velocity"] = torch.zeros(n, 3, 3, dtype=template_batch.positions.dtype, device=template_batch.device)
        return st

    def pre_update(self, batch: Batch) -> None:
        s = self._state
        m = batch.num_graphs

        def step_cell(cell_force: torch.Tensor) -> None:
            idx = torch.arange(m, device=batch.device, dtype=torch.int32).repeat_interleave(3)
            cell = batch.cell.reshape(m * 3, 3)
            a, d, nsi = s["alpha"].clone(), s["dt"].clone(), s["nsteps_inc"].clone()
            fire2_step_coord(cell, s["cell_velocity"].reshape(m * 3, 3), cell_force.reshape(m * 3, 3), idx, a, d, nsi,
                             **self.hp)

        self._cell_step(batch, step_cell)
        super().pre_update(batch)
