# SPDX-License-Identifier: Apache-2.0
"""Lennard-Jones model over the dense neighbour matrix (reference ``nvalchemi/models/lj.py:82-510``).

``E = sum_pairs 4 eps [(sigma/r)^12 - (sigma/r)^6] S(r)`` with a C2 switch ``S`` on the last ``switch_width`` before the
cutoff.  Energies, forces and the virial are produced directly by the kernel (no autograd); the stress is
``-virial / volume``.  Works with full or half neighbour lists, on CPU and CUDA.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


def lj_energy_forces_virial_batch(positions, cells, neighbor_matrix, neighbor_matrix_shifts, num_neighbors, batch_idx,
                                  fill_value, epsilon, sigma, cutoff, switch_width, half_list, num_systems):
    """Per-atom energies ``[N]``, forces ``[N,3]`` and per-system virials ``[B,9]``."""
    if _native.require(positions):
        return _nops.lj_energy_forces_virial_batch(positions.detach().contiguous(), cells.contiguous(),
                                                   neighbor_matrix.contiguous(), neighbor_matrix_shifts.contiguous(),
                                                   num_neighbors.contiguous(), batch_idx.to(torch.int32), int(fill_value),
                                                   float(epsilon), float(sigma), float(cutoff), float(switch_width),
                                                   bool(half_list), int(num_systems))
    return _lj_torch(positions, cells, neighbor_matrix, neighbor_matrix_shifts, num_neighbors, batch_idx, epsilon, sigma,
                     cutoff, switch_width, half_list, num_systems)


def _lj_torch(pos, cells, nm, shifts, num, batch_idx, eps, sigma, rc, sw, half, nsys):
    n, k = nm.shape
    valid = torch.arange(k, device=nm.device)[None] < num[:, None].clamp_max(k)
    i = torch.arange(n, device=nm.device)[:, None].expand(n, k)[valid]
    j = nm[valid].long()
    b = batch_idx.long()
    p = pos.detach().double().requires_grad_(True)
    d = p[j] + torch.einsum("ei,eij->ej", shifts[valid].double(), cells.double()[b[i]]) - p[i]
    strain = torch.zeros(nsys, 3, 3, dtype=torch.float64, device=pos.device, requires_grad=True)
    d = d + torch.einsum("ei,eij->ej", d, 0.5 * (strain + strain.transpose(1, 2))[b[i]])
    r = d.norm(dim=-1)
    sr6 = (sigma / r) ** 6
    u = 4 * eps * (sr6 * sr6 - sr6)
    if sw > 0:
        x = ((r - (rc - sw)) / sw).clamp(0, 1)
        u = u * (1 - x ** 3 * (10 - 15 * x + 6 * x * x))
    u = torch.where(r < rc, u, torch.zeros_like(u)) * (1.0 if half else 0.5)
    e_atom = torch.zeros(n, dtype=torch.float64, device=pos.device).index_add_(0, i, u)
    g, gs = torch.autograd.grad(u.sum(), [p, strain])
    return e_atom.detach().to(pos.dtype), (-g).to(pos.dtype), (-gs).reshape(nsys, 9).to(pos.dtype)


class LennardJonesModelWrapper(nn.Module, BaseModelMixin):
    def __init__(self, epsilon: float, sigma: float, cutoff: float, switch_width: float = 0.0,
                 half_list: bool = False) -> None:
        super().__init__()
        self.epsilon, self.sigma, self.cutoff = float(epsilon), float(sigma), float(cutoff)
        self.switch_width, self.half_list = float(switch_width), bool(half_list)
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress", "virial", "atomic_energies"}),
            optional_inputs=frozenset({"cell", "pbc", "neighbor_matrix_shifts"}), supports_pbc=True,
            neighbor_config=NeighborConfig(cutoff=self.cutoff, format=NeighborListFormat.MATRIX, half_list=half_list),
            active_outputs={"energy", "forces"})

    def forward(self, data: Any, **kwargs: Any) -> dict:
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        batch_idx = data.batch_idx if hasattr(data, "batch_idx") else torch.zeros(
            data.positions.shape[0], dtype=torch.int32, device=data.positions.device)
        cell, _ = _nb.cell_and_pbc(data) if hasattr(data, "num_graphs") else (
            torch.eye(3, device=data.positions.device).reshape(1, 3, 3), None)
        nm = data.neighbor_matrix
        sh = getattr(data, "neighbor_matrix_shifts", None)
        if sh is None:
            sh = torch.zeros(nm.shape + (3,), dtype=torch.int32, device=nm.device)
        n = data.positions.shape[0]
        e_atom, forces, virial = lj_energy_forces_virial_batch(
            data.positions, cell.to(data.positions.dtype), nm, sh, data.num_neighbors, batch_idx, n, self.epsilon,
            self.sigma, self.cutoff, self.switch_width, self.half_list, nb)
        energy = torch.zeros(nb, dtype=torch.float64, device=e_atom.device).index_add_(0, batch_idx.long(), e_atom.double())
        out = {"energy": energy.to(e_atom.dtype).unsqueeze(-1), "forces": forces, "atomic_energies": e_atom,
               "virial": virial.reshape(nb, 3, 3)}
        vol = torch.linalg.det(cell.double()).abs().clamp_min(1e-30).to(e_atom.dtype)
        out["stress"] = -out["virial"] / vol[:, None, None]
        return self.adapt_output(out, data)

    def checkpoint_spec(self) -> dict:
        return {"cls": "nvalchemi_toolkit_b200.models.lj.LennardJonesModelWrapper",
                "config": {"epsilon": self.epsilon, "sigma": self.sigma, "cutoff": self.cutoff,
                           "switch_width": self.switch_width, "half_list": self.half_list}}

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed.spec import SPEC_LJ_HALO

        return SPEC_LJ_HALO
