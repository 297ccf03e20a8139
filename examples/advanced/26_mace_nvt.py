# SPDX-License-Identifier: Apache-2.0
"""NVT Langevin MD with a MACE model (random weights: the point is the workflow, not the physics).

On a CUDA device the float32 wrapper in eval mode runs the native kernels (fused convolution, grouped tf32 GEMMs,
symmetric contraction); on CPU, in float64 or in training mode the differentiable PyTorch statement of the same network
runs instead (`MACE._use_native` makes the choice per call)."""
import argparse

import torch

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import DynamicsStage, NVTLangevin, _ops
from nvalchemi_toolkit_b200.models.mace import MACEWrapper

ap = argparse.ArgumentParser()
ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
ap.add_argument("--cells", type=int, default=2)
ap.add_argument("--steps", type=int, default=10)
ap.add_argument("--channels", type=int, default=16)
args = ap.parse_args()

torch.manual_seed(0)
batch = build("fcc_cu", args.cells, device=args.device)
wrapper = MACEWrapper(atomic_numbers=[29], channels=args.channels, r_max=5.0, avg_num_neighbors=40.0).to(args.device).eval()
wrapper.model_config.active_outputs = {"energy", "forces"}
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 300.0, batch.batch_idx, random_seed=0)
dyn = NVTLangevin(wrapper, dt=1.0, temperature=300.0, friction=0.01, random_seed=1, hooks=wrapper.make_neighbor_hooks())


class Log:
    frequency, stage = 5, DynamicsStage.AFTER_STEP

    def __call__(self, ctx, stage):
        b = ctx.batch
        ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs)
        t = _ops.compute_temperature(ke, b.num_nodes_per_graph)
        print(f"step {ctx.step_count:3d}  E_pot = {float(b.energy):10.4f} eV  T = {float(t):6.1f} K", flush=True)


dyn.register_hook(Log())
dyn.run(batch, n_steps=args.steps)
native = wrapper.model._use_native(batch.positions, wrapper.training)
print(f"{batch.num_nodes} atoms on {args.device}: {'native sm_100a kernels' if native else 'PyTorch path'}")
