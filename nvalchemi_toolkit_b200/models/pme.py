# SPDX-License-Identifier: Apache-2.0
"""Smooth particle-mesh Ewald (reference ``nvalchemi/models/pme.py:83-939``).

Real-space sum, self term, neutralising background and slab correction are shared with the direct Ewald wrapper
(``_CoulombBase`` in ``models/ewald.py``); this module adds the reciprocal part on a mesh: B-spline charge assignment
(``pme_spread`` kernel), FFT, multiplication with the influence function (B-spline moduli), inverse FFT and the gather of
potential and field at the atoms (``pme_gather`` kernel), in ``models/_electrostatics.py::recip_mesh``.  The mesh is chosen
from ``mesh_spacing`` or, by default, from the requested accuracy (``pme_mesh_dims``); the set-up (mesh dimensions and
moduli) is cached per system and rebuilt when the cell changes."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.models import _electrostatics as es
from nvalchemi_toolkit_b200.models._electrostatics import bspline_moduli, pme_mesh_dims
from nvalchemi_toolkit_b200.models.ewald import _CoulombBase

__all__ = ["PMEModelWrapper", "pme_mesh_dims", "bspline_moduli"]


class PMEModelWrapper(_CoulombBase):
    """Smooth particle-mesh Ewald (B-spline order ``spline_order``, mesh from ``mesh_spacing`` or the accuracy)."""

    method = "pme"

    def __init__(self, cutoff: float = 10.0, accuracy: float = 1e-6, alpha: float | None = None, spline_order: int = 5,
                 mesh_spacing: float | None = None, mesh_dims: tuple[int, int, int] | None = None, **kw: Any) -> None:
        super().__init__(cutoff=cutoff, accuracy=accuracy, alpha=alpha, spline_order=spline_order,
                         mesh_spacing=mesh_spacing, mesh_dims=mesh_dims, **kw)
        self.order, self.mesh_spacing, self.mesh_dims = int(spline_order), mesh_spacing, mesh_dims

    def _build_setup(self, cell: torch.Tensor) -> Any:
        dims = tuple(self.mesh_dims) if self.mesh_dims is not None else es.pme_mesh_dims(
            cell, self.alpha, self.accuracy, self.mesh_spacing, self.order)
        moduli = tuple(es.bspline_moduli(n, self.order).to(cell.device) for n in dims)
        return dims, moduli

    def _recip(self, positions, charges, cell, setup, a0, a1, weights, reduce):
        dims, moduli = setup
        return es.recip_mesh(positions, charges, cell, self.alpha, dims, self.order, moduli, a0, a1, weights, reduce)
