# SPDX-License-Identifier: Apache-2.0
"""Relax -> heat -> production in ONE fused workflow: ``fire + langevin + nve`` builds a ``FusedStage`` whose per-system
status selects the integrator (0: FIRE until fmax, 1: Langevin for 40 steps, 2: NVE for 40 steps, 3: done).  All systems
share every model evaluation; a stage-timing hook reports where the step time goes."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, NVE, ConvergenceHook, NVTLangevin, _ops
from nvalchemi_toolkit_b200.hooks import StageTimingHook
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

torch.manual_seed(0)
batch = Batch.from_data_list([systems.argon_cluster(n, noise=0.12, seed=n, dtype=torch.float64) for n in (13, 19, 27, 38)])
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=10.0)
relax = FIRE(model, dt=1.0, convergence_hook=ConvergenceHook.from_fmax(5e-3))
heat = NVTLangevin(model, dt=2.0, temperature=30.0, friction=0.05, random_seed=3, n_steps=40)
produce = NVE(model, dt=2.0, n_steps=40)
workflow = relax + heat + produce
log = Path(tempfile.mkdtemp()) / "stage_times.csv"
timing = StageTimingHook("detailed", log_path=log)
workflow.register_hook(timing)
for h in model.make_neighbor_hooks():
    workflow.register_hook(h)
workflow.run(batch, n_steps=400)
status = batch.status.reshape(-1).tolist()
ke = _ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, batch.num_graphs)
temps = _ops.compute_temperature(ke, batch.num_nodes_per_graph).tolist()
print("final status per system:", status, "| fused steps:", workflow.step_count)
print("temperatures after production:", [round(t, 1) for t in temps], "K")
print("stage timing rows:", len(timing.rows), "->", log)
assert all(s == 3 for s in status)
