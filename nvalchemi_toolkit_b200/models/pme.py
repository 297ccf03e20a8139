# SPDX-License-Identifier: Apache-2.0
"""Particle-mesh Ewald wrapper (reference ``nvalchemi/models/pme.py:83-939``); the implementation shares its real-space,
self, background and slab terms with the Ewald wrapper and lives beside it."""
from nvalchemi_toolkit_b200.models._electrostatics import bspline_moduli, pme_mesh_dims
from nvalchemi_toolkit_b200.models.ewald import PMEModelWrapper

__all__ = ["PMEModelWrapper", "pme_mesh_dims", "bspline_moduli"]
