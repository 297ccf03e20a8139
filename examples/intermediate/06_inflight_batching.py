# SPDX-License-Identifier: Apache-2.0
"""Relax-then-equilibrate many systems with a fused two-stage workflow and inflight batching: a system that finishes
stage 0 moves to stage 1 in the same batch, a system that finishes stage 1 goes to the sink and its slot is refilled
from the sampler, so the device batch stays full."""
import torch

from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, NVE, ConvergenceHook, HostMemory, SizeAwareSampler
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper


class Clusters:
    """Any object with ``__len__``, ``__getitem__ -> (AtomicData, meta)`` and ``get_metadata(i) -> (atoms, edges)``."""

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
sampler = SizeAwareSampler(Clusters([8, 21, 13, 34, 5, 16, 27, 9, 12, 30]), max_atoms=64, max_batch_size=4)
sink = HostMemory()
relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(0.05))
md = NVE(model, dt=0.5, n_steps=20)
workflow = relax + md                      # FusedStage: status 0 runs FIRE, status 1 runs NVE, status 2 is done
workflow.sampler, workflow.sinks = sampler, [sink]
workflow.run()
done = sink.read()
print("finished systems:", done.num_graphs, "| sizes:", sorted(done.num_nodes_list))
print("fused steps:", workflow.step_count, "| sampler exhausted:", sampler.exhausted)
