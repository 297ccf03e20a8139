# SPDX-License-Identifier: Apache-2.0
"""NPT (Nose-Hoover chain + MTK barostat) on a domain-decomposed system:

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/31_npt_domain_parallel.py

Thermostat and barostat are global controllers: kinetic energy, kinetic tensor and virial are summed over the ranks
before the chain and the cell update, so every rank integrates the same cell trajectory and scales its own atoms.  A
compressed argon crystal expands towards zero pressure; the cell and the volume agree on all ranks by construction."""
import os

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel
from nvalchemi_toolkit_b200.dynamics import NPT, _ops
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

if "RANK" in os.environ:
    dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
rank = dist.get_rank() if dist.is_initialized() else 0

batch = build("fcc_cu", 4, a=5.15, z=18, dtype=torch.float64)            # compressed: equilibrium is near 5.3 A
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 40.0, batch.batch_idx, random_seed=0)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
model.model_config.active_outputs = {"energy", "forces", "stress"}
dyn = NPT(model, dt=2.0, temperature=40.0, pressure=0.0, barostat_time=200.0, thermostat_time=50.0)
dp = DomainParallel(dyn, DomainConfig(cutoff=8.0, skin=1.0))
v0 = float(torch.linalg.det(batch.cell.reshape(3, 3)))
sharded = dp.run(batch, n_steps=60)
v1 = float(torch.linalg.det(sharded.owned.cell.reshape(3, 3)))
print(f"rank {rank}: {sharded.n_owned} owned atoms; volume {v0:.1f} -> {v1:.1f} A^3 "
      f"({dp.num_rebuilds} re-partitions as the box grew)", flush=True)
assert v1 > v0
if dist.is_initialized():
    dist.destroy_process_group()
