# SPDX-License-Identifier: Apache-2.0
"""Writing a hook and a convergence criterion of your own.

A hook is any object with ``frequency``, ``stage`` and ``__call__(ctx, stage)``; a criterion is a dictionary
``{key, threshold, reduce_op / custom_op}`` evaluated per system and AND-ed with the others.  Here a relaxation stops
when the largest force AND the energy change between consecutive steps are both small."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, DynamicsStage
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper


class EnergyChange:
    """Stores ``|E_t - E_{t-1}|`` per system on the batch so that a criterion can read it."""

    frequency, stage = 1, DynamicsStage.AFTER_COMPUTE

    def __init__(self):
        self.last = None
        self.history = []

    def __call__(self, ctx, stage):
        e = ctx.batch.energy.detach().reshape(-1)
        change = torch.full_like(e, float("inf")) if self.last is None else (e - self.last).abs()
        self.last = e.clone()
        ctx.batch.add_key("energy_change", change.reshape(-1, 1), level="system", overwrite=True)
        self.history.append(float(e.sum()))


batch = Batch.from_data_list([systems.argon_cluster(n, noise=0.15, seed=n) for n in (10, 14, 19)])
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
tracker = EnergyChange()
criteria = [{"key": "forces", "threshold": 5e-3, "reduce_op": "norm", "reduce_dims": -1},
            {"key": "energy_change", "threshold": 1e-6}]
opt = FIRE(model, dt=0.3, convergence_hook=ConvergenceHook(criteria), hooks=model.make_neighbor_hooks() + [tracker])
opt._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
opt.compute(batch)
opt.run(batch, n_steps=600)
print(f"stopped after {opt.step_count} steps; energy {tracker.history[0]:.4f} -> {tracker.history[-1]:.4f} eV; "
      f"fmax = {float(batch.forces.norm(dim=-1).max()):.2e} eV/A")
