# SPDX-License-Identifier: Apache-2.0
"""Two workflows on one domain-decomposed system: a FIRE relaxation that stops when EVERY rank's atoms are converged
(one small AND-reduction per step), then Langevin MD continued from the relaxed, still sharded state.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/distributed/22_relax_then_md_domain_parallel.py

Run without ``torchrun`` the script starts two CPU ranks itself.  On GPUs with the native MACE the same code uses the
peer-memory transport automatically."""
import os
import sys

import torch
import torch.distributed as dist


def main() -> None:
    from nvalchemi_toolkit_b200.benchmark import build
    from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel
    from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, NVTLangevin, _ops
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

    rank = dist.get_rank()
    batch = build("fcc_cu", 4, a=5.26, z=18, noise=0.12, dtype=torch.float64)
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
    cfg = DomainConfig(cutoff=8.5, skin=1.0)
    with DomainParallel(FIRE(model, dt=0.5, convergence_hook=ConvergenceHook.from_fmax(0.01)), cfg) as relax:
        sharded = relax.run(batch, n_steps=400)
        steps = relax.dynamics.step_count
        fmax = float(sharded.owned.forces.norm(dim=-1).max())
    print(f"rank {rank}: relaxation stopped after {steps} steps (converged everywhere: {relax.converged}), "
          f"local fmax {fmax:.4f} eV/A", flush=True)
    owned = sharded.owned
    _ops.initialize_velocities(owned.velocities, owned.atomic_masses, 40.0, owned.batch_idx, random_seed=3 + rank)
    md = DomainParallel(NVTLangevin(model, dt=2.0, temperature=40.0, friction=0.02, random_seed=9), cfg)
    md.run(sharded, n_steps=25)
    full = md.gather(dst=0)
    if rank == 0:
        print(f"after MD: {full.num_nodes} atoms gathered, E = {float(full.energy):.4f} eV", flush=True)


def _rank(rank: int, world: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29642", RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    main()
    dist.destroy_process_group()


if __name__ == "__main__":
    if "RANK" in os.environ:
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
        main()
        dist.destroy_process_group()
    else:
        import torch.multiprocessing as mp

        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        mp.spawn(_rank, args=(2,), nprocs=2)
