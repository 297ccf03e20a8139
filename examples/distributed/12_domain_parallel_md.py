# SPDX-License-Identifier: Apache-2.0
"""Domain-decomposed MD of one system over ranks (any backend):

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/distributed/12_domain_parallel_md.py

Each rank integrates the atoms inside its box; ghost atoms come from the neighbours, atoms that leave a box migrate
with all their fields, hooks with ``HookScope.RANK_ZERO`` see the gathered system.  Without ``torchrun`` the script runs
as a single rank (periodic images are then the only ghosts)."""
import os

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel, HookScope
from nvalchemi_toolkit_b200.dynamics import DynamicsStage, NVTLangevin, _ops
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

if "RANK" in os.environ:
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(backend)
rank = dist.get_rank() if dist.is_initialized() else 0
device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and dist.is_initialized() else "cpu"

batch = build("fcc_cu", 5, device=device, a=5.26, z=18, dtype=torch.float64)      # the same on every rank
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 80.0, batch.batch_idx, random_seed=0)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
dyn = NVTLangevin(model, dt=2.0, temperature=80.0, friction=0.02, random_seed=5)
dp = DomainParallel(dyn, DomainConfig(cutoff=8.5, skin=1.0))


class PrintEnergy:
    frequency, stage = 10, DynamicsStage.AFTER_STEP

    def __call__(self, ctx, stage):
        b = ctx.batch
        print(f"step {ctx.step_count:3d}: {b.num_nodes} atoms, E = {float(b.energy):.4f} eV", flush=True)


dp.register_hook(PrintEnergy(), scope=HookScope.RANK_ZERO)
sharded = dp.run(batch, n_steps=30)
print(f"rank {rank}: owns {sharded.n_owned} atoms, {sharded.n_ghost} ghosts, "
      f"{dp.num_rebuilds} re-partitions, {sharded.num_migrated} migrations", flush=True)
if dist.is_initialized():
    dist.destroy_process_group()
