# SPDX-License-Identifier: Apache-2.0
"""A harmonic restraint added to a model's forces with ``BiasedPotentialHook``: the cluster's centre is pulled towards a
target point while Langevin dynamics runs, and the bias energy is reported next to the model energy."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import DynamicsStage, NVTLangevin, _ops
from nvalchemi_toolkit_b200.hooks.bias import BiasedPotentialHook
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

torch.manual_seed(0)
batch = Batch.from_data_list([systems.argon_cluster(24, noise=0.05, seed=1)])
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 30.0, batch.batch_idx, random_seed=2)
target = batch.positions.mean(0) + torch.tensor([3.0, 0.0, 0.0])  # 3 A away from where the cluster starts
k_spring = 0.5  # eV / A^2


def restraint(b):
    centre = b.positions.mean(0)
    d = centre - target
    energy = 0.5 * k_spring * (d * d).sum()
    forces = (-k_spring * d / b.num_nodes).expand_as(b.positions)  # dE/dr_i = k d / N for every atom
    return energy.reshape(1, 1), forces


model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
dyn = NVTLangevin(model, dt=2.0, temperature=30.0, friction=0.05, random_seed=3,
                  hooks=model.make_neighbor_hooks() + [BiasedPotentialHook(restraint, stage=DynamicsStage.AFTER_COMPUTE)])
start = float((batch.positions.mean(0) - target).norm())
dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
dyn.compute(batch)
dyn.run(batch, n_steps=400)
end = float((batch.positions.mean(0) - target).norm())
print(f"distance of the cluster centre from the target: {start:.2f} A -> {end:.2f} A")
assert end < start
