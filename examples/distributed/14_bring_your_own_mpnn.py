# SPDX-License-Identifier: Apache-2.0
"""Bring your own message-passing network and run it domain-decomposed WITHOUT touching its code:

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/14_bring_your_own_mpnn.py

The network below is plain PyTorch (``h[src]`` gathers, ``index_add_`` scatters) and knows nothing about ranks.  With
``MLIPSpec(refresh_per_layer=True)`` the ghost layer is one cutoff deep however many layers the network has: inside the
distributed forward a dispatch mode notices every scatter that produces a node tensor and refreshes the ghost rows
from their owners before the next gather (differentiably, so forces come out right).  Without ``torchrun`` the script
runs as one rank whose only ghosts are periodic images."""
import os

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import build
from nvalchemi_toolkit_b200.distributed import (Consolidation, DistributedModel, DomainConfig, MLIPSpec, ShardedBatch,
                                                ShardTensor)
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.neighbors import compute_neighbors

CUTOFF = 4.0


class TinyMPNN(torch.nn.Module):
    def __init__(self, width: int = 16, layers: int = 3) -> None:
        super().__init__()
        self.emb = torch.nn.Embedding(100, width)
        self.mix = torch.nn.ModuleList(torch.nn.Linear(width, width) for _ in range(layers))
        self.out = torch.nn.Linear(width, 1)

    def forward(self, z, pos, src, dst, shifts, batch, n_graphs):
        h = self.emb(z)
        d = (pos[src] + shifts - pos[dst]).norm(dim=-1, keepdim=True)
        w = torch.exp(-d) * (d < CUTOFF)
        for lin in self.mix:
            h = h + torch.tanh(torch.zeros_like(h).index_add_(0, dst, lin(h)[src] * w))
        return torch.zeros(n_graphs, dtype=pos.dtype, device=pos.device).index_add_(0, batch, self.out(h).squeeze(-1))


class TinyWrapper(torch.nn.Module, BaseModelMixin):
    """The usual wrapper contract: neighbour matrix in, energy and autograd forces out."""

    def __init__(self) -> None:
        super().__init__()
        torch.manual_seed(0)
        self.net = TinyMPNN().double()
        self.model_config = ModelConfig(outputs=frozenset({"energy", "forces"}),
                                        neighbor_config=NeighborConfig(cutoff=CUTOFF, format=NeighborListFormat.MATRIX))

    def forward(self, data, **kw):
        pos = data.positions.detach().requires_grad_()
        nm, num = data.neighbor_matrix.long(), data.num_neighbors.long()
        valid = torch.arange(nm.shape[1], device=nm.device)[None, :] < num[:, None]
        dst = torch.arange(nm.shape[0], device=nm.device)[:, None].expand_as(nm)[valid]
        src = nm[valid]
        cell = data.cell[data.batch_idx.long()[dst]].to(pos.dtype)
        shifts = torch.einsum("ei,eij->ej", data.neighbor_matrix_shifts[valid].to(pos.dtype), cell)
        n_graphs = int(data.cell.shape[0])
        e = self.net(data.atomic_numbers.long(), pos, src, dst, shifts, data.batch_idx.long(), n_graphs)
        (g,) = torch.autograd.grad(e.sum(), pos)
        return {"energy": e.detach().reshape(n_graphs, 1), "forces": -g}

    def distribution_spec(self, strategy=None):
        return MLIPSpec("tiny_mpnn", message_passes=3, consolidation=Consolidation.WEIGHTED_ENERGY, refresh_per_layer=True)


if "RANK" in os.environ:
    dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
rank = dist.get_rank() if dist.is_initialized() else 0

batch = build("fcc_cu", 4, a=3.61, z=29, dtype=torch.float64)                      # the same on every rank
model = TinyWrapper()
cfg = DomainConfig(cutoff=CUTOFF, skin=0.0)

spec = model.distribution_spec()
sharded = ShardedBatch.from_batch(batch, cfg, spec)
dm = DistributedModel(model, cfg, spec=spec)
out = dm(sharded)
forces = ShardTensor(out["forces"], sharded).full_tensor()                         # global atom order, on every rank

deep = ShardedBatch.from_batch(batch, cfg, spec.with_(refresh_per_layer=False))    # ghosts three cutoffs deep instead
ref = Batch.from_data_list([batch.get_data(0)])
compute_neighbors(ref, config=model.model_config.neighbor_config)
single = model(ref)
err = float((forces - single["forces"]).abs().max())
print(f"rank {rank}: {sharded.n_owned} owned + {sharded.n_ghost} ghosts (a 3-cutoff halo would need {deep.n_ghost}); "
      f"{dm.last_dispatch_stats.get('refreshes', 0)} ghost refreshes; E = {float(out['energy']):.6f} eV; "
      f"max |F - F_single| = {err:.2e}", flush=True)
assert err < 1e-8

# Had the wrapper declared nothing, one traced single-process forward proposes the spec: it counts the neighbour
# aggregations on the way to the energy (three here) and sees that the model sums over atoms itself.
from nvalchemi_toolkit_b200.distributed.infer_spec import infer_spec  # noqa: E402

proposed, seen = infer_spec(model, ref)
if rank == 0:
    print(f"trace: {seen.describe()}\nproposed: message_passes={proposed.message_passes}, "
          f"consolidation={proposed.consolidation.value}, refresh_per_layer={proposed.refresh_per_layer}", flush=True)
assert proposed.message_passes == spec.message_passes and proposed.refresh_per_layer
if dist.is_initialized():
    dist.destroy_process_group()
