# SPDX-License-Identifier: Apache-2.0
"""A new integrator in a few lines: subclass ``BaseDynamics``, implement ``pre_update`` (before the forces are
evaluated) and ``post_update`` (after).  The example is a velocity-Verlet step with a Berendsen-style velocity rescale;
everything else (hooks, stage fusion with ``+``, pipelines with ``|``, inflight batching) is inherited."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.dynamics import BaseDynamics, DynamicsStage, _ops
from nvalchemi_toolkit_b200.dynamics._units import fs_to_internal_time
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper


class BerendsenNVT(BaseDynamics):
    __needs_keys__ = {"forces"}
    __provides_keys__ = {"positions", "velocities"}

    def __init__(self, model, dt, temperature, coupling_time, **kw):
        super().__init__(model=model, **kw)
        self.dt, self.tau, self.temperature = fs_to_internal_time(dt), fs_to_internal_time(coupling_time), temperature

    def _init_state(self, batch):
        m = batch.num_graphs
        self._state = {"dt": torch.full((m,), self.dt, dtype=batch.positions.dtype, device=batch.device)}

    def pre_update(self, batch):
        _ops.vv_position_update(batch.positions, batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"],
                                batch.batch_idx)

    def post_update(self, batch):
        _ops.vv_velocity_finalize(batch.velocities, batch.forces, batch.atomic_masses, self._state["dt"], batch.batch_idx)
        ke = _ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, batch.num_graphs)
        t_now = _ops.compute_temperature(ke, batch.num_nodes_per_graph).clamp_min(1e-6)
        scale = torch.sqrt(1.0 + (self.dt / self.tau) * (self.temperature / t_now - 1.0))
        _ops.velocity_rescale(batch.velocities, scale.to(batch.velocities.dtype), batch.batch_idx)


batch = Batch.from_data_list([systems.fcc(3, a=5.3, z=18, noise=0.05, seed=0)])
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 10.0, batch.batch_idx, random_seed=0)
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
dyn = BerendsenNVT(model, dt=2.0, temperature=60.0, coupling_time=100.0, hooks=model.make_neighbor_hooks())
dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
dyn.compute(batch)
dyn.run(batch, n_steps=300)
ke = _ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, 1)
print(f"temperature after 300 steps: {float(_ops.compute_temperature(ke, batch.num_nodes_per_graph)):.1f} K (target 60 K)")
