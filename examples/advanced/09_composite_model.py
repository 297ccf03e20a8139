# SPDX-License-Identifier: Apache-2.0
"""MACE + DFT-D3(BJ) + particle-mesh Ewald as one model: additive groups, shared neighbour lists, one NVT run.

The three members have cutoffs 5, 10 and 9 A; the pipeline builds one neighbour list at 10 A for the two long-ranged
members (9 A is within the 1.5x sharing ratio) and a separate 5 A list for MACE."""
import argparse

import torch

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import NVTLangevin, _ops
from nvalchemi_toolkit_b200.models.dftd3 import DFTD3ModelWrapper, DFTD3Parameters
from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper
from nvalchemi_toolkit_b200.models.mace import MACEWrapper
from nvalchemi_toolkit_b200.models.pipeline import PipelineGroup, PipelineModelWrapper

ap = argparse.ArgumentParser()
ap.add_argument("--device", default="cpu")
ap.add_argument("--size", type=int, default=2)
ap.add_argument("--steps", type=int, default=5)
args = ap.parse_args()

torch.manual_seed(0)
batch = build("nacl", args.size, device=args.device)          # carries node_charges (+1 / -1)
mace = MACEWrapper(atomic_numbers=[11, 17], channels=16, r_max=5.0, avg_num_neighbors=18.0).to(args.device)
d3 = DFTD3ModelWrapper("pbe", parameters=DFTD3Parameters.synthetic(20), cutoff=10.0)  # placeholder tables, see the class docs
pme = PMEModelWrapper(cutoff=9.0, accuracy=1e-5)
model = PipelineModelWrapper([PipelineGroup([mace]), PipelineGroup([d3]), PipelineGroup([pme])])
model.model_config.active_outputs = {"energy", "forces"}
print(model)
print("neighbour sources (cutoffs):", [s.cutoff for s in model._sources])
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 300.0, batch.batch_idx, random_seed=0)
dyn = NVTLangevin(model, dt=1.0, temperature=300.0, friction=0.01, random_seed=3, hooks=model.make_neighbor_hooks())
dyn.run(batch, n_steps=args.steps)
print(f"{batch.num_nodes} atoms, {args.steps} steps: E = {float(batch.energy):.4f} eV, "
      f"fmax = {float(batch.forces.norm(dim=-1).max()):.3f} eV/A")
