# SPDX-License-Identifier: Apache-2.0
"""NVT Langevin dynamics of solid argon: the kinetic temperature relaxes from 20 K to the 80 K bath and then fluctuates
around it; a batch of two independent systems runs in the same kernels (per-system dt, temperature, friction)."""
import argparse

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark.systems import fcc
from nvalchemi_toolkit_b200.dynamics import DynamicsStage, NVTLangevin, _ops
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

ap = argparse.ArgumentParser()
ap.add_argument("--device", default="cpu")
ap.add_argument("--steps", type=int, default=300)
args = ap.parse_args()

batch = Batch.from_data_list([fcc(3, a=5.26, z=18, noise=0.02, seed=s, dtype=torch.float64) for s in (0, 1)], device=args.device)
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 20.0, batch.batch_idx, random_seed=1)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
dyn = NVTLangevin(model, dt=2.0, temperature=80.0, friction=0.05, random_seed=11, hooks=model.make_neighbor_hooks())
temps = []


class Thermometer:
    frequency, stage = 10, DynamicsStage.AFTER_STEP

    def __call__(self, ctx, stage):
        b = ctx.batch
        ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs)
        temps.append(_ops.compute_temperature(ke, b.num_nodes_per_graph).tolist())


dyn.register_hook(Thermometer())
dyn.run(batch, n_steps=args.steps)
first, last = temps[0], [sum(t[i] for t in temps[-10:]) / 10 for i in range(2)]
print(f"temperature after 10 steps: {first[0]:.1f} K / {first[1]:.1f} K; mean of the last 100 steps: {last[0]:.1f} K / {last[1]:.1f} K")
assert all(40.0 < t < 130.0 for t in last), "the thermostat did not bring the systems to the bath temperature"
