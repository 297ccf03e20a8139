# SPDX-License-Identifier: Apache-2.0
"""A graph transformer (attention over neighbours) run domain-decomposed through the deep-halo route:

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/30_bring_your_own_graph_transformer.py

With ``MLIPSpec(message_passes=L, refresh_per_layer=False)`` every rank keeps ghosts ``L`` cutoffs deep and evaluates the
unmodified network on owned + ghost atoms: whatever the layers do (attention normalisation, gating, residuals), the
energy of every owned atom is exact, because its whole receptive field is local.  The framework sums the owned node
energies, differentiates, and returns the ghost rows' gradients to their owners.  Nothing is intercepted, so this route
needs no knowledge of the model's operators; it pays with a deeper ghost layer than the per-layer refresh route."""
import os

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.distributed import Consolidation, DistributedModel, DomainConfig, MLIPSpec, ShardedBatch, ShardTensor
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.neighbors import compute_neighbors

CUTOFF, LAYERS = 4.0, 2


class AttentionLayer(torch.nn.Module):
    def __init__(self, width: int, heads: int) -> None:
        super().__init__()
        self.q, self.k, self.v = (torch.nn.Linear(width, width, bias=False) for _ in range(3))
        self.rbf = torch.nn.Linear(8, heads)
        self.out = torch.nn.Linear(width, width)
        self.heads = heads

    def forward(self, h, src, dst, dist_e):
        n, w = h.shape
        hd = w // self.heads
        q, k, v = (f(h).view(n, self.heads, hd) for f in (self.q, self.k, self.v))
        centers = torch.linspace(0.5, CUTOFF, 8, dtype=h.dtype, device=h.device)
        basis = torch.exp(-4.0 * (dist_e[:, None] - centers) ** 2)
        envelope = 0.5 * (torch.cos(torch.pi * dist_e / CUTOFF) + 1.0) * (dist_e < CUTOFF)       # smooth cutoff
        logits = torch.tanh((q[dst] * k[src]).sum(-1) / hd ** 0.5 + self.rbf(basis))            # bounded: exp is safe
        weight = torch.exp(logits) * envelope[:, None]
        norm = torch.zeros(n, self.heads, dtype=h.dtype, device=h.device).index_add_(0, dst, weight) + 1.0
        msg = torch.zeros(n, self.heads, hd, dtype=h.dtype, device=h.device).index_add_(0, dst, weight[..., None] * v[src])
        return h + self.out((msg / norm[..., None]).reshape(n, w))


class GraphTransformer(torch.nn.Module, BaseModelMixin):
    def __init__(self, width: int = 16, heads: int = 4) -> None:
        super().__init__()
        torch.manual_seed(0)
        self.emb = torch.nn.Embedding(100, width)
        self.layers = torch.nn.ModuleList(AttentionLayer(width, heads) for _ in range(LAYERS))
        self.readout = torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.SiLU(), torch.nn.Linear(width, 1))
        self.double()
        self.model_config = ModelConfig(outputs=frozenset({"energy", "forces", "atomic_energies"}),
                                        neighbor_config=NeighborConfig(cutoff=CUTOFF, format=NeighborListFormat.MATRIX))

    def forward(self, data, **kw):
        pos = data.positions.detach().requires_grad_()
        nm, num = data.neighbor_matrix.long(), data.num_neighbors.long()
        valid = torch.arange(nm.shape[1], device=nm.device)[None, :] < num[:, None]
        dst = torch.arange(nm.shape[0], device=nm.device)[:, None].expand_as(nm)[valid]
        src = nm[valid]
        cell = data.cell[data.batch_idx.long()[dst]].to(pos.dtype)
        shifts = torch.einsum("ei,eij->ej", data.neighbor_matrix_shifts[valid].to(pos.dtype), cell)
        d = (pos[src] + shifts - pos[dst]).norm(dim=-1)
        h = self.emb(data.atomic_numbers.long())
        for layer in self.layers:
            h = layer(h, src, dst, d)
        e_atom = self.readout(h).squeeze(-1)
        weights = getattr(data, "energy_weights", None)          # 1 for owned atoms, 0 for ghosts (absent in a plain batch)
        e_sum = e_atom if weights is None else e_atom * weights.to(e_atom.dtype)
        n_graphs = int(data.cell.shape[0])
        energy = torch.zeros(n_graphs, dtype=pos.dtype, device=pos.device).index_add_(0, data.batch_idx.long(), e_sum)
        (g,) = torch.autograd.grad(energy.sum(), pos)
        return {"energy": energy.detach().reshape(n_graphs, 1), "forces": -g, "atomic_energies": e_atom.detach()}

    def distribution_spec(self, strategy=None):
        return MLIPSpec("graph_transformer", message_passes=LAYERS, consolidation=Consolidation.WEIGHTED_ENERGY)


if "RANK" in os.environ:
    dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
rank = dist.get_rank() if dist.is_initialized() else 0

batch = build("nacl", 3, dtype=torch.float64)                                       # the same on every rank
model = GraphTransformer()
cfg = DomainConfig(cutoff=CUTOFF, skin=0.0)
spec = model.distribution_spec()
sharded = ShardedBatch.from_batch(batch, cfg, spec)
out = DistributedModel(model, cfg, spec=spec)(sharded)
forces = ShardTensor(out["forces"], sharded).full_tensor()

ref = Batch.from_data_list([batch.get_data(0)])
compute_neighbors(ref, config=model.model_config.neighbor_config)
single = model(ref)
err_f = float((forces - single["forces"]).abs().max())
err_e = abs(float(out["energy"]) - float(single["energy"]))
print(f"rank {rank}: {sharded.n_owned} owned + {sharded.n_ghost} ghosts ({LAYERS} x {CUTOFF} A deep); "
      f"E = {float(out['energy']):.6f} eV (single process {float(single['energy']):.6f}); max |F - F_single| = {err_f:.2e}", flush=True)
assert err_f < 1e-8 and err_e < 1e-8
if dist.is_initialized():
    dist.destroy_process_group()
