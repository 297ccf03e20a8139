# SPDX-License-Identifier: Apache-2.0
"""Monitoring a two-rank stage pipeline: who is busy, how many systems are in flight, what each stage costs.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/34_pipeline_monitoring.py

Every rank registers its own hooks on its own stage: a ``StageTimingHook`` (per-stage wall time, written per rank), a
``LoggingHook`` with a custom scalar (systems in the active batch) and a small occupancy probe.  At the end the per-rank
summaries are gathered so rank 0 can print one table: the place to see an unbalanced pipeline (a starving MD rank or a
relaxation rank that cannot keep up)."""
import os
import tempfile
from pathlib import Path

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, DemoDynamics, DynamicsStage, HostMemory, SizeAwareSampler
from nvalchemi_toolkit_b200.dynamics.hooks.library import LoggingHook
from nvalchemi_toolkit_b200.hooks import StageTimingHook
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper

if "RANK" not in os.environ:
    raise SystemExit("start this example with torchrun --nproc-per-node 2")
dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
rank = dist.get_rank()
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


class Occupancy:
    """Counts steps and the systems they advanced (a hook is any object with frequency / stage / __call__)."""

    frequency, stage = 1, DynamicsStage.AFTER_STEP

    def __init__(self):
        self.steps = self.system_steps = 0

    def __call__(self, ctx, stage):
        self.steps += 1
        self.system_steps += ctx.batch.num_graphs


torch.manual_seed(0)
model = DemoModelWrapper()
out = Path(tempfile.mkdtemp())
sampler = SizeAwareSampler(Clusters([8, 21, 13, 34, 5, 16, 9, 27]), max_atoms=64, max_batch_size=3)
sink = HostMemory()
relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(0.05), sampler=sampler, device_type=device_type, max_batch_size=3)
md = DemoDynamics(model, n_steps=10, dt=0.05, sinks=[sink], device_type=device_type, max_batch_size=8)
mine = relax if rank == 0 else md
occupancy = Occupancy()
timing = StageTimingHook("step", log_path=out / f"timing_rank{rank}.csv")
log = LoggingHook(backend="csv", frequency=5, log_path=out / f"scalars_rank{rank}.csv",
                  custom_scalars={"systems_in_batch": lambda ctx: float(ctx.batch.num_graphs)})
for hook in (occupancy, timing, log):
    mine.register_hook(hook)
pipe = relax | md
pipe.setup()
with log:
    pipe.run(max_iterations=500)
done = sink.read()
step_ms = [r.get("step_ms", r.get("total_ms", 0.0)) for r in timing.rows]
summary = {"rank": rank, "role": "relax (FIRE)" if rank == 0 else "md", "stage_steps": occupancy.steps,
           "system_steps": occupancy.system_steps, "iterations": pipe.iterations,
           "mean_step_ms": sum(step_ms) / max(1, len(step_ms)), "finished_here": 0 if done is None else done.num_graphs}
gathered = [None] * dist.get_world_size()
dist.all_gather_object(gathered, summary)
if rank == 0:
    print(f"{'rank':>4} {'role':<14} {'steps':>6} {'system-steps':>12} {'idle iterations':>15} {'finished':>8}")
    for s in gathered:
        print(f"{s['rank']:>4} {s['role']:<14} {s['stage_steps']:>6} {s['system_steps']:>12} "
              f"{s['iterations'] - s['stage_steps']:>15} {s['finished_here']:>8}")
    print("per-rank logs in", out)
    assert gathered[1]["finished_here"] == 8
dist.destroy_process_group()
