# SPDX-License-Identifier: Apache-2.0
"""Guard rails for long runs: clamp runaway forces, stop on NaNs, watch the energy drift of an NVE trajectory, and log
per-system scalars to CSV in the background."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import NVE, DynamicsStage, _ops
from nvalchemi_toolkit_b200.dynamics.hooks.library import (EnergyDriftMonitorHook, LoggingHook, MaxForceClampHook,
                                                           NaNDetectorHook)
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

batch = Batch.from_data_list([systems.fcc(3, a=5.3, z=18, noise=0.05, seed=s, dtype=torch.float64) for s in (0, 1)])
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 40.0, batch.batch_idx, random_seed=0)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
log = Path(tempfile.mkdtemp()) / "md.csv"
drift = EnergyDriftMonitorHook(threshold=1e-4, metric="per_atom_per_step")
hooks = model.make_neighbor_hooks() + [MaxForceClampHook(max_force=5.0), NaNDetectorHook(), drift,
                                       LoggingHook(backend="csv", frequency=10, log_path=log)]
dyn = NVE(model, dt=2.0, hooks=hooks)
dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
dyn.compute(batch)
dyn.run(batch, n_steps=100)
rows = log.read_text().strip().splitlines() if log.exists() else []
print(f"100 NVE steps of {batch.num_graphs} systems; log rows: {len(rows)}; positions finite: {bool(torch.isfinite(batch.positions).all())}")
