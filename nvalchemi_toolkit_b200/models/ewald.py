# SPDX-License-Identifier: Apache-2.0
"""Ewald summation and particle-mesh Ewald model wrappers.

Reference: ``nvalchemi/models/ewald.py:77-944`` and ``nvalchemi/models/pme.py:83-939``: point-charge electrostatics of
periodic systems from per-atom ``node_charges``; ``alpha``, k-vectors / mesh and spline moduli are cached per system
and recomputed when the cell changes; forces and stresses are analytic; the energy is differentiable with respect to
the charges, positions and cell (the analytic potentials, forces and virial are injected as gradients), so a
charge-predicting model upstream trains through it; ``slab_correction`` handles systems periodic in x and y only.
Under domain decomposition the reciprocal sum runs over owned charges (``energy_weights``) and the structure factors
or the mesh are all-reduced.
"""
from __future__ import annotations

import math
from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.models import _electrostatics as es
from nvalchemi_toolkit_b200.models._utils import cell_cache_needs_update
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat


class _CoulombEnergy(torch.autograd.Function):
    """Energy ``[B]`` whose backward injects analytic derivatives: ``dE/dr = -F``, ``dE/dq = phi`` and a cell gradient
    that makes ``dE/d(strain)`` of the affine strain construction equal ``-W``."""

    @staticmethod
    def forward(ctx: Any, positions, charges, cells, batch_idx, energy, forces, virial, phi, weights=None):
        ctx.save_for_backward(positions.detach(), cells.detach(), batch_idx, forces, virial, phi)
        ctx.weights = weights
        return energy.clone()

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor):
        positions, cells, batch_idx, forces, virial, phi = ctx.saved_tensors
        b = batch_idx.long()
        g = grad.reshape(-1)
        gp = -forces * g[b][:, None]
        gq = phi * g[b]
        if ctx.weights is not None:
            # one rank's share of a decomposed system: F_i and phi_i of an OWNED atom are already the derivatives of the
            # whole system's energy; a ghost row's derivatives are accounted for on the rank that owns the atom
            w = ctx.weights.to(gp.dtype)
            gp, gq = gp * w[:, None], gq * w
        # dE/d(strain) = sum_i r_i (x) dE/dr_i + cell^T dE/dcell = -W  =>  dE/dcell = cell^-T (-W + sum_i r_i (x) F_i)
        rf = torch.zeros_like(virial).index_add_(0, b, positions[:, :, None] * forces[:, None, :])
        gc = torch.linalg.solve(cells.transpose(1, 2), (-virial + rf)) * g[:, None, None]
        return gp, gq, gc, None, None, None, None, None, None


class _CoulombBase(nn.Module, BaseModelMixin):
    method = "ewald"

    def __init__(self, cutoff: float = 10.0, accuracy: float = 1e-6, alpha: float | None = None,
                 coulomb_constant: float = es.COULOMB_EV_A, slab_correction: bool = False,
                 charge_key: str = "node_charges", **mesh: Any) -> None:
        super().__init__()
        self.cutoff, self.accuracy, self.ke = float(cutoff), float(accuracy), float(coulomb_constant)
        a, kc = es.estimate_ewald_parameters(self.cutoff, self.accuracy)
        self.alpha = float(alpha) if alpha is not None else a
        self.k_cutoff = 2.0 * self.alpha * math.sqrt(-math.log(self.accuracy))
        self.slab_correction, self.charge_key, self.mesh_opts = bool(slab_correction), charge_key, mesh
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress", "virial", "atomic_energies", "electrostatic_potential"}),
            required_inputs=frozenset({charge_key, "cell"}), optional_inputs=frozenset({"pbc", "neighbor_matrix_shifts"}),
            supports_pbc=True, needs_pbc=True,
            neighbor_config=NeighborConfig(cutoff=self.cutoff, format=NeighborListFormat.MATRIX, half_list=False),
            active_outputs={"energy", "forces"})
        self._cache: dict[int, tuple[torch.Tensor, Any]] = {}

    # ---- per-system reciprocal set-up, cached on the cell --------------------------------------------------------
    def _setup(self, sys_idx: int, cell: torch.Tensor) -> Any:
        hit = self._cache.get(sys_idx)
        if hit is not None and not cell_cache_needs_update(hit[0], cell):
            return hit[1]
        value = self._build_setup(cell)
        self._cache[sys_idx] = (cell.detach().clone(), value)
        return value

    def _build_setup(self, cell: torch.Tensor) -> Any:
        return es.generate_k_vectors(cell, self.k_cutoff).to(cell.device)

    def _recip(self, positions, charges, cell, setup, a0, a1, weights, reduce):
        return es.recip_direct(positions, charges, cell, setup, self.alpha, a0, a1, weights, reduce)

    def invalidate_cache(self) -> None:
        self._cache.clear()

    # ---- evaluation ---------------------------------------------------------------------------------------------
    def compute(self, data: Any) -> dict[str, torch.Tensor]:
        pos, q = data.positions, getattr(data, self.charge_key)
        q = q.reshape(-1)
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        n = pos.shape[0]
        batch_idx = data.batch_idx if hasattr(data, "batch_idx") else torch.zeros(n, dtype=torch.int32, device=pos.device)
        ptr = data.batch_ptr.tolist() if hasattr(data, "batch_ptr") else [0, n]
        cells = data.cell.reshape(nb, 3, 3)
        weights = getattr(data, "energy_weights", None)
        dd = getattr(data, "_dd", None)  # (group, world) when the batch is one rank's padded share of a system
        reduce = None
        if dd is not None and dd[1] > 1:
            import torch.distributed as dist

            from nvalchemi_toolkit_b200.parallel.symmetric import peer_reducer

            # structure factors / charge meshes are summed through peer memory where the ranks share NVLink (ordered
            # float64 peer loads between two flag barriers); elsewhere through the library collective
            reduce = peer_reducer(dd[0], pos.device)
            if reduce is None:
                def reduce(t: torch.Tensor, _g: Any = dd[0]) -> torch.Tensor:
                    dist.all_reduce(t, group=_g)
                    return t
        alpha = torch.full((nb,), self.alpha, dtype=torch.float64, device=pos.device)
        e_atom, forces, virial, phi = es.real_space(pos, q, cells, data.neighbor_matrix,
                                                    getattr(data, "neighbor_matrix_shifts", None), data.num_neighbors,
                                                    batch_idx, alpha, self.cutoff, False, nb)
        forces, virial, phi = forces.double(), virial.double(), phi.double()
        qd = q.detach().double()
        wq = qd if weights is None else qd * weights.double()
        for s in range(nb):
            a0, a1 = ptr[s], ptr[s + 1]
            cell = cells[s]
            vol = float(torch.linalg.det(cell.detach().double()).abs())
            _, f_s, w_s, phi_s = self._recip(pos, q, cell, self._setup(s, cell), a0, a1, weights, reduce)
            forces[a0:a1] += f_s
            phi[a0:a1] += phi_s
            scale = 1.0 if reduce is None else 1.0 / dd[1]  # every rank holds the same reciprocal virial
            virial[s] += scale * w_s
            qtot = wq[a0:a1].sum()
            if reduce is not None:
                qtot = reduce(qtot.clone())
            phi[a0:a1] += -2.0 * self.alpha / math.sqrt(math.pi) * qd[a0:a1] - math.pi / (vol * self.alpha ** 2) * qtot
            # the neutralising background has E = -pi Q^2 / (2 V a^2): dE/d(strain_aa) = +pi Q^2 / (2 V a^2)
            virial[s] -= scale * torch.eye(3, dtype=torch.float64, device=pos.device) * math.pi * qtot ** 2 / (
                2.0 * vol * self.alpha ** 2)
            if self.slab_correction:
                r = pos.detach().double()[a0:a1]
                m = (wq[a0:a1, None] * r).sum(0)  # dipole moment of the cell
                if reduce is not None:
                    m = reduce(m.clone())
                phi[a0:a1] += 4.0 * math.pi / vol * m[2] * r[:, 2]
                forces[a0:a1, 2] += -4.0 * math.pi / vol * m[2] * qd[a0:a1]
                e_slab = 2.0 * math.pi / vol * m[2] * m[2]
                ez = torch.zeros(3, dtype=torch.float64, device=pos.device)
                ez[2] = 1.0
                corr = torch.eye(3, dtype=torch.float64, device=pos.device) * e_slab - 2.0 * math.pi / vol * m[2] * (
                    ez[:, None] * m[None, :] + m[:, None] * ez[None, :])
                virial[s] += scale * corr
        e_atom = 0.5 * qd * phi  # E = 1/2 sum_i q_i phi_i (real, reciprocal, self, background, slab are all quadratic)
        if weights is not None:
            e_atom = e_atom * weights.double()
        energy = torch.zeros(nb, dtype=torch.float64, device=pos.device).index_add_(0, batch_idx.long(), e_atom)
        ke = self.ke
        return {"energy": ke * energy, "forces": ke * forces, "virial": ke * virial, "phi": ke * phi,
                "atomic_energies": ke * e_atom, "cells": cells, "batch_idx": batch_idx}

    def forward(self, data: Any, **kwargs: Any) -> dict:
        r = self.compute(data)
        pos, q = data.positions, getattr(data, self.charge_key).reshape(-1)
        dtype = pos.dtype
        energy = r["energy"]
        cells = data.cell.reshape(-1, 3, 3)
        if torch.is_grad_enabled() and (pos.requires_grad or q.requires_grad or cells.requires_grad):
            energy = _CoulombEnergy.apply(pos.double() if pos.dtype != torch.float64 else pos,
                                          q.double() if q.dtype != torch.float64 else q,
                                          cells.double() if cells.dtype != torch.float64 else cells,
                                          r["batch_idx"], energy, r["forces"], r["virial"], r["phi"],
                                          getattr(data, "energy_weights", None))
        vol = torch.linalg.det(r["cells"].detach().double()).abs().clamp_min(1e-30)
        out = {"energy": energy.to(dtype).unsqueeze(-1), "forces": r["forces"].to(dtype),
               "virial": r["virial"].to(dtype), "stress": (-r["virial"] / vol[:, None, None]).to(dtype),
               "atomic_energies": r["atomic_energies"].to(dtype), "electrostatic_potential": r["phi"].to(dtype)}
        return self.adapt_output(out, data)

    def checkpoint_spec(self) -> dict:
        cfg = {"cutoff": self.cutoff, "accuracy": self.accuracy, "alpha": self.alpha, "coulomb_constant": self.ke,
               "slab_correction": self.slab_correction, "charge_key": self.charge_key, **self.mesh_opts}
        return {"cls": f"{type(self).__module__}.{type(self).__name__}", "config": cfg}

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed.spec import SPEC_EWALD_REAL_HALO

        return SPEC_EWALD_REAL_HALO


class EwaldModelWrapper(_CoulombBase):
    """Direct reciprocal sum: cost ``O(N K)``; exact to the chosen accuracy; best below ~10^4 atoms."""


def __getattr__(name: str) -> Any:
    """``PMEModelWrapper`` moved to :mod:`nvalchemi_toolkit_b200.models.pme`; the old import path keeps working."""
    if name == "PMEModelWrapper":
        from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper

        return PMEModelWrapper
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
