# SPDX-License-Identifier: Apache-2.0
"""NPT with full cell coupling: a sheared argon crystal relaxes its shear stress when the barostat may change the cell
angles (``pressure_coupling="triclinic"``), which the per-axis modes cannot do."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import NPT, DynamicsStage, _ops
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
for mode in ("anisotropic", "triclinic"):
    batch = Batch.from_data_list([systems.fcc(3, a=5.3, z=18, noise=0.05, seed=0, dtype=torch.float64)])
    shear = torch.eye(3, dtype=torch.float64)
    shear[0, 1] = shear[1, 0] = 0.03
    batch["positions"] = batch.positions @ shear
    cell = batch.cell.reshape(-1, 3, 3)
    cell.copy_(cell @ shear)
    _ops.initialize_velocities(batch.velocities, batch.atomic_masses, 20.0, batch.batch_idx, random_seed=1)
    dyn = NPT(model, dt=2.0, temperature=20.0, pressure=0.0, barostat_time=150.0, thermostat_time=50.0,
              pressure_coupling=mode, hooks=model.make_neighbor_hooks())
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    before = float(batch.stress.reshape(3, 3)[0, 1])
    dyn.run(batch, n_steps=150)
    c = batch.cell.reshape(3, 3)
    angle = torch.rad2deg(torch.acos((c[0] @ c[1]) / (c[0].norm() * c[1].norm())))
    print(f"{mode:12s}: shear stress {before:+.5f} -> {float(batch.stress.reshape(3, 3)[0, 1]):+.5f} eV/A^3, "
          f"angle(a, b) = {float(angle):.2f} deg")
