# SPDX-License-Identifier: Apache-2.0
"""Custom hooks, safety hooks and the reporting stack on a Langevin run."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import DynamicsStage, NVTLangevin, _ops
from nvalchemi_toolkit_b200.dynamics.hooks.library import MaxForceClampHook, NaNDetectorHook
from nvalchemi_toolkit_b200.hooks import WrapPeriodicHook
from nvalchemi_toolkit_b200.hooks.reporting import JSONLReporter, ReportingOrchestrator, RichReporter
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper


class MeanSquareDisplacement:
    """A hook is any object with ``frequency``, ``stage`` and ``__call__(ctx, stage)``."""

    frequency, stage = 10, DynamicsStage.AFTER_STEP

    def __init__(self):
        self.start, self.values = None, []

    def __call__(self, ctx, stage):
        pos = ctx.batch.positions
        if self.start is None:
            self.start = pos.clone()
        self.values.append((ctx.step_count, float((pos - self.start).pow(2).sum(-1).mean())))


batch = build("fcc_cu", 3, a=5.26, z=18, dtype=torch.float64)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 60.0, batch.batch_idx, random_seed=0)
out = Path(tempfile.mkdtemp())
msd = MeanSquareDisplacement()
report = ReportingOrchestrator([RichReporter(layout="dynamics", title="argon, Langevin 60 K"),
                                JSONLReporter(out / "metrics.jsonl")], frequency=25)
dyn = NVTLangevin(model, dt=2.0, temperature=60.0, friction=0.02, random_seed=1,
                  hooks=model.make_neighbor_hooks() + [NaNDetectorHook(), MaxForceClampHook(max_force=5.0), msd, report])
with report:
    dyn.run(batch, n_steps=100)
print("mean square displacement:", ", ".join(f"{s}: {v:.3f}" for s, v in msd.values[::3]), "A^2")
print("metrics written to", out / "metrics.jsonl")
