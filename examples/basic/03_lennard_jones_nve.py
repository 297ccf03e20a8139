# SPDX-License-Identifier: Apache-2.0
"""NVE molecular dynamics of solid argon with the Lennard-Jones kernel; energy conservation check."""
import argparse

import torch

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import NVE, _ops
from nvalchemi_toolkit_b200.dynamics.hooks.library import EnergyDriftMonitorHook, LoggingHook
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

ap = argparse.ArgumentParser()
ap.add_argument("--device", default="cpu")
ap.add_argument("--cells", type=int, default=4)
ap.add_argument("--steps", type=int, default=100)
args = ap.parse_args()

batch = build("fcc_cu", args.cells, device=args.device, a=5.26, z=18, dtype=torch.float64)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 40.0, batch.batch_idx, random_seed=0)
rows = []
log = LoggingHook(backend="custom", frequency=20, writer_fn=lambda step, r: rows.append((step, r[0])))
drift = EnergyDriftMonitorHook(threshold=1e-5, frequency=10)  # eV per atom per step; warns when exceeded
dyn = NVE(model, dt=2.0, hooks=model.make_neighbor_hooks() + [log, drift])
dyn.run(batch, n_steps=args.steps)  # hooks that are context managers are opened and closed by run()
for step, r in rows:
    print(f"step {step:4d}  E_pot {r['energy']:.4f} eV  T {r['temperature']:.1f} K  fmax {r['fmax']:.3f} eV/A")
print("energy drift per atom per step:", f"{float(drift.last_drift.max()):.2e}", "eV")
