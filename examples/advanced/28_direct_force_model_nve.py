# SPDX-License-Identifier: Apache-2.0
"""NVE with a graph network that takes an edge list with cell offsets (the UMA / fairchem calling convention).

``UMAWrapper`` builds ``edge_index`` + ``cell_offsets`` from the package's neighbour matrix, calls the network with a
``pos / atomic_numbers / cell / batch / edge_index / cell_offsets`` dictionary and differentiates the returned energy.
The fairchem package is not needed: any module with that calling convention can be wrapped, here a two-layer
message-passing stand-in."""
import torch
from torch import nn

from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.dynamics import NVE, _ops
from nvalchemi_toolkit_b200.models.uma import UMAWrapper


class TinyEdgeNet(nn.Module):
    num_layers = 2

    def __init__(self, width: int = 8) -> None:
        super().__init__()
        self.embed = nn.Embedding(100, width)
        self.mix = nn.ModuleList(nn.Linear(width, width) for _ in range(self.num_layers))
        self.out = nn.Linear(width, 1)

    def forward(self, d):
        src, dst = d["edge_index"]
        off = torch.einsum("ei,eij->ej", d["cell_offsets"].to(d["pos"].dtype), d["cell"][d["batch"][dst]])
        r = (d["pos"][src] + off - d["pos"][dst]).norm(dim=-1)
        w = (0.5 * (torch.cos(torch.pi * r / 6.0) + 1.0) * torch.exp(-r / 2.0)).unsqueeze(-1)   # smooth to zero at 6 A
        h = self.embed(d["atomic_numbers"]).to(d["pos"].dtype)
        for lin in self.mix:
            h = h + torch.tanh(lin(torch.zeros_like(h).index_add_(0, dst, w * h[src])))
        e_atom = self.out(h).squeeze(-1)
        return {"energy": torch.zeros(d["cell"].shape[0], dtype=e_atom.dtype).index_add_(0, d["batch"], e_atom)}


torch.manual_seed(0)
batch = build("fcc_cu", 2, dtype=torch.float64)
model = UMAWrapper(TinyEdgeNet().double(), cutoff=6.0)
model.model_config.active_outputs = {"energy", "forces"}
_ops.initialize_velocities(batch.velocities, batch.atomic_masses, 200.0, batch.batch_idx, random_seed=0)
dyn = NVE(model, dt=1.0, hooks=model.make_neighbor_hooks())
e0 = None
for _ in range(4):
    dyn.run(batch, n_steps=5)
    tot = float(batch.energy) + float(_ops.compute_kinetic_energy(batch.velocities, batch.atomic_masses, batch.batch_idx, 1))
    e0 = tot if e0 is None else e0
    print(f"step {dyn.step_count:3d}  E_tot = {tot:.6f} eV  (drift {tot - e0:+.1e})")
assert abs(tot - e0) < 1e-3
