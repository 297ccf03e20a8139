# SPDX-License-Identifier: Apache-2.0
"""Node (graph) partition of ONE system that has no useful spatial order: a gas-phase cluster whose atoms are stored in
random order.  Every rank owns a contiguous index block, evaluates only the edges whose receiver it owns, and asks the
other blocks for the sender rows it needs (before every message-passing layer).

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/21_graph_partition.py

Run without ``torchrun`` the script starts two CPU ranks itself."""
import os
import sys

import torch
import torch.distributed as dist


def main() -> None:
    from nvalchemi_toolkit_b200 import Batch
    from nvalchemi_toolkit_b200.benchmark import systems
    from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel, StrategyKind
    from nvalchemi_toolkit_b200.dynamics import NVE, _ops
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

    rank, world = dist.get_rank(), dist.get_world_size()
    d = systems.argon_cluster(120, noise=0.05, seed=0)
    perm = torch.randperm(d.positions.shape[0], generator=torch.Generator().manual_seed(1))
    d.__dict__["positions"] = d.positions[perm].contiguous()  # no spatial order left
    batch = Batch.from_data_list([d])
    _ops.initialize_velocities(batch.velocities, batch.atomic_masses, 30.0, batch.batch_idx, random_seed=0)
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
    cfg = DomainConfig(cutoff=8.5, skin=1.0, strategy=StrategyKind.GRAPH_PARTITION)
    dp = DomainParallel(NVE(model, dt=2.0), cfg)
    sharded = dp.run(batch, n_steps=20)
    print(f"rank {rank}/{world}: owns atoms [{int(sharded.global_ids[0])}, {int(sharded.global_ids[-1])}], "
          f"{sharded.halo.edges_owned} edges, {sharded.n_ghost} sender rows from other blocks", flush=True)
    full = dp.gather(dst=0)
    if rank == 0:
        print(f"gathered {full.num_nodes} atoms, E = {float(full.energy):.4f} eV", flush=True)


def _rank(rank: int, world: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29641", RANK=str(rank), WORLD_SIZE=str(world))
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
