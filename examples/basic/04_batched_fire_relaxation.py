# SPDX-License-Identifier: Apache-2.0
"""Relax many small clusters at once with FIRE; each system stops when its own forces converge."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

clusters = [systems.argon_cluster(n, noise=0.15, seed=n, dtype=torch.float64) for n in (13, 19, 38, 55)]
batch = Batch.from_data_list(clusters)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=10.0)
opt = FIRE(model, dt=1.0, hooks=model.make_neighbor_hooks(), convergence_hook=ConvergenceHook.from_fmax(2e-3))
opt.run(batch, n_steps=400)
fmax = torch.zeros(batch.num_graphs, dtype=torch.float64).scatter_reduce(
    0, batch.batch_idx.long(), batch.forces.norm(dim=-1), "amax", include_self=False)
for n, e, f in zip(batch.num_nodes_list, batch.energy.reshape(-1).tolist(), fmax.tolist()):
    print(f"Ar{n:<3d} E = {e:9.4f} eV   fmax = {f:.1e} eV/A")
print("steps taken:", opt.step_count)
