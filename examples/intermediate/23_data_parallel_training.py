# SPDX-License-Identifier: Apache-2.0
"""Data-parallel training: every rank trains on its own batches and ``FusedGradAllReduceHook`` averages the gradients
(bucketed; on GPUs the buckets live in peer-mapped memory and their reductions overlap the backward pass; on CPU ranks a
``torch.distributed`` all-reduce of the same flat buffer is used).

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/intermediate/23_data_parallel_training.py

Run without ``torchrun`` the script starts two CPU ranks itself."""
import os
import sys

import torch
import torch.distributed as dist


def main() -> None:
    from nvalchemi_toolkit_b200 import Batch
    from nvalchemi_toolkit_b200.benchmark import systems
    from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper
    from nvalchemi_toolkit_b200.training import EnergyMSELoss, ForceMSELoss, OptimizerConfig, TrainingStrategy
    from nvalchemi_toolkit_b200.training.hooks import FusedGradAllReduceHook

    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    teacher = DemoModelWrapper()

    def labelled(n, seed):
        d = systems.argon_cluster(n, noise=0.2, seed=seed)
        out = teacher(Batch.from_data_list([d]))
        d.__dict__["energy"], d.__dict__["forces"] = out["energy"].detach().reshape(1, 1), out["forces"].detach()
        return d

    mine = [labelled(6 + i % 5, 1000 * rank + i) for i in range(16)]           # each rank sees different structures
    loader = [Batch.from_data_list(mine[i:i + 4]) for i in range(0, 16, 4)]
    torch.manual_seed(1)
    strategy = TrainingStrategy(DemoModelWrapper(), OptimizerConfig(kwargs={"lr": 3e-3}),
                                loss_fn=EnergyMSELoss() + 10.0 * ForceMSELoss(), num_epochs=5, devices=["cpu"],
                                hooks=[FusedGradAllReduceHook(bucket_mb=0.01)])
    strategy.run(loader)
    checksum = sum(float(p.detach().double().sum()) for p in strategy.models["main"].parameters())
    sums = [None] * world
    dist.all_gather_object(sums, checksum)
    if rank == 0:
        print(f"{world} ranks, {strategy.step_count} steps, loss {float(strategy.last_losses['total_loss']):.5f}; "
              f"replicas identical: {max(sums) - min(sums) < 1e-9}", flush=True)


def _rank(rank: int, world: int) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29643", RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    main()
    dist.destroy_process_group()


if __name__ == "__main__":
    if "RANK" in os.environ:
        dist.init_process_group("gloo")
        main()
        dist.destroy_process_group()
    else:
        import torch.multiprocessing as mp

        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        mp.spawn(_rank, args=(2,), nprocs=2)
