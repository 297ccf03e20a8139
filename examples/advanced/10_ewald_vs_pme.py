# SPDX-License-Identifier: Apache-2.0
"""Madelung energy of rock salt with Ewald and PME at several accuracies; stress and potentials."""
import math
from types import SimpleNamespace

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.models._electrostatics import COULOMB_EV_A
from nvalchemi_toolkit_b200.models.ewald import EwaldModelWrapper
from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper
import torch

exact = -1.7475645946 * COULOMB_EV_A / (5.64 / 2)
for cls in (EwaldModelWrapper, PMEModelWrapper):
    for acc in (1e-4, 1e-6, 1e-8):
        batch = build("nacl", 2, noise=0.0, dtype=torch.float64)
        model = cls(cutoff=5.5, accuracy=acc)
        model.model_config.active_outputs = {"energy", "forces", "stress", "electrostatic_potential"}
        for h in model.make_neighbor_hooks():
            h(SimpleNamespace(batch=batch), None)
        out = model(batch)
        per_pair = float(out["energy"]) / (batch.num_nodes / 2)
        print(f"{cls.__name__:18s} accuracy {acc:.0e}: E/pair = {per_pair:.7f} eV  (error {abs(per_pair - exact):.1e}), "
              f"potential at Na = {float(out['electrostatic_potential'][0]):.5f} V, "
              f"pressure = {-float(out['stress'][0].diagonal().mean()) * 160.21766:.3f} GPa")
print(f"exact Madelung energy per pair: {exact:.7f} eV")
