# SPDX-License-Identifier: Apache-2.0
"""Relax atoms and cell of a strained Lennard-Jones crystal under zero pressure with variable-cell FIRE."""
import torch

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import ConvergenceHook, FIREVariableCell
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

batch = build("fcc_cu", 3, a=5.6, z=18, noise=0.02, dtype=torch.float64)     # 6 % too large
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
model.model_config.active_outputs = {"energy", "forces", "stress"}
a0 = float(batch.cell[0, 0, 0]) / 3
opt = FIREVariableCell(model, dt=1.0, hooks=model.make_neighbor_hooks(), convergence_hook=ConvergenceHook.from_fmax(5e-4))
opt._call_hooks(type(opt)._stage_type.BEFORE_COMPUTE, batch)
opt.compute(batch)                                   # forces and stress of the starting structure
opt.run(batch, n_steps=300)
a1 = float(batch.cell[0, 0, 0]) / 3
print(f"lattice constant {a0:.3f} -> {a1:.3f} A in {opt.step_count} steps; "
      f"residual pressure {-float(batch.stress[0].diagonal().mean()) * 160.21766:.4f} GPa")
