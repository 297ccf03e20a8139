# SPDX-License-Identifier: Apache-2.0
"""Two dynamics stages on two ranks: rank 0 relaxes structures, rank 1 runs MD on the ones that converged.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/13_stage_pipeline.py

Graduated systems travel between ranks with point-to-point messages that overlap the next step."""
import os

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, DemoDynamics, HostMemory, SizeAwareSampler
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper

if "RANK" not in os.environ:
    raise SystemExit("start this example with torchrun --nproc-per-node 2")
dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
device_type = "cuda" if torch.cuda.is_available() else "cpu"


class Clusters:
    def __init__(self, sizes):
        self.items = [systems.argon_cluster(n, noise=0.1, seed=i) for i, n in enumerate(sizes)]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i], {}

    def get_metadata(self, i):
        return self.items[i].positions.shape[0], 0


torch.manual_seed(0)
model = DemoModelWrapper()
sampler = SizeAwareSampler(Clusters([8, 21, 13, 34, 5, 16]), max_atoms=64, max_batch_size=3)
sink = HostMemory()
relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(0.05), sampler=sampler, device_type=device_type,
             max_batch_size=3)
md = DemoDynamics(model, n_steps=10, dt=0.05, sinks=[sink], device_type=device_type, max_batch_size=8)
pipe = relax | md
pipe.setup()
pipe.run(max_iterations=500)
done = sink.read()
print(f"rank {dist.get_rank()}: {pipe.iterations} iterations, finished here: {0 if done is None else done.num_graphs}", flush=True)
dist.destroy_process_group()
