# SPDX-License-Identifier: Apache-2.0
"""A short-range network that predicts partial charges, wired into Ewald electrostatics (the AIMNet2 + Coulomb pattern).

``PipelineStep(wire={"charges": "node_charges"})`` hands the first model's ``charges`` output to the second model's
``node_charges`` input; the group runs under autograd, so the forces include the response of the predicted charges
(d E_coul / d q * d q / d r).  The AIMNet2 package is not required: the wrapper adapts any module with AIMNet2's calling
convention, here a small stand-in network."""
import torch
from torch import nn

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import NVE, _ops
from nvalchemi_toolkit_b200.models.aimnet2 import AIMNet2Wrapper
from nvalchemi_toolkit_b200.models.ewald import EwaldModelWrapper
from nvalchemi_toolkit_b200.models.pipeline import PipelineGroup, PipelineModelWrapper, PipelineStep


class TinyChargeNet(nn.Module):
    """AIMNet2 calling convention: padded neighbour matrix ``nbmat`` (index N = padding row), ``coord`` with one padding
    row, ``mol_idx``, per-molecule ``charge``; returns ``energy`` per molecule and ``charges`` per atom (+ padding)."""

    cutoff = 4.5

    def __init__(self) -> None:
        super().__init__()
        self.scale = nn.Parameter(torch.tensor(0.3))

    def forward(self, d):
        coord, nbmat = d["coord"], d["nbmat"]
        n = coord.shape[0] - 1
        r = (coord[nbmat[:n]] + d["shifts"][:n] - coord[:n, None]).norm(dim=-1)
        w = torch.exp(-r) * (nbmat[:n] < n)
        sign = torch.where(d["numbers"][:n] == 11, 1.0, -1.0).to(coord.dtype)
        q = sign * torch.tanh(self.scale * w.sum(-1))
        mol = d["mol_idx"][:n]
        q = q - torch.zeros(d["charge"].shape[0], dtype=q.dtype).index_add_(0, mol, q)[mol] / torch.bincount(mol)[mol]
        e = torch.zeros(d["charge"].shape[0], dtype=coord.dtype).index_add_(0, mol, 0.05 * w.sum(-1))
        return {"energy": e, "charges": torch.cat([q, q.new_zeros(1)])}


torch.manual_seed(0)
batch = build("nacl", 2, dtype=torch.float64)
net = AIMNet2Wrapper(TinyChargeNet())
net.model_config.active_outputs = {"energy", "charges"}
coulomb = EwaldModelWrapper(cutoff=8.0, accuracy=1e-6)
model = PipelineModelWrapper([PipelineGroup([PipelineStep(net, wire={"charges": "node_charges"}), coulomb], use_autograd=True)])
model.model_config.active_outputs = {"energy", "forces"}
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 300.0, batch.batch_idx, random_seed=0)
dyn = NVE(model, dt=0.5, hooks=model.make_neighbor_hooks())
e0 = None
for block in range(4):
    dyn.run(batch, n_steps=5)
    ke = float(_ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, 1))
    tot = float(batch.energy) + ke
    e0 = tot if e0 is None else e0
    print(f"step {dyn.step_count:3d}  E_pot = {float(batch.energy):9.4f}  E_tot = {tot:9.4f} eV  (drift {tot - e0:+.2e})")
assert abs(tot - e0) < 5e-3, "energy drift: forces and energy are inconsistent"
