# SPDX-License-Identifier: Apache-2.0
"""AIMNet2 / UMA adapters driven by stand-in networks with the external calling conventions."""
from types import SimpleNamespace

import torch
from torch import nn

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.models.aimnet2 import AIMNet2Wrapper
from nvalchemi_toolkit_b200.models.uma import UMAWrapper
from tests.helpers import fcc_supercell


class _FakeAIMNet(nn.Module):
    cutoff = 4.0

    def forward(self, d):
        coord, nbmat = d["coord"], d["nbmat"]
        n = coord.shape[0] - 1
        rj = coord[nbmat[:n]] + d["shifts"][:n]
        r = (rj - coord[:n, None]).norm(dim=-1)
        mask = nbmat[:n] < n
        e_atom = (torch.exp(-r) * mask).sum(-1)
        mol = d["mol_idx"][:n]
        energy = torch.zeros(d["charge"].shape[0], dtype=coord.dtype).index_add_(0, mol, e_atom)
        return {"energy": energy, "charges": torch.cat([torch.tanh(e_atom - 1.0), e_atom.new_zeros(1)]),
                "aim": torch.cat([e_atom[:, None].expand(n, 4), e_atom.new_zeros(1, 4)])}


class _FakeUMA(nn.Module):
    num_layers = 2

    def forward(self, d):
        src, dst = d["edge_index"]
        off = torch.einsum("ei,eij->ej", d["cell_offsets"], d["cell"][d["batch"][dst]])
        r = (d["pos"][src] + off - d["pos"][dst]).norm(dim=-1)
        e = torch.zeros(d["cell"].shape[0], dtype=r.dtype).index_add_(0, d["batch"][dst], 0.5 * torch.exp(-r))
        return {"energy": e}


def _neighbors(model, batch):
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)


def _pair_reference(batch, cutoff):
    pos = batch.positions.clone().requires_grad_(True)
    cell = batch.cell.reshape(3, 3)
    s = torch.stack(torch.meshgrid(*[torch.arange(-1, 2)] * 3, indexing="ij"), -1).reshape(-1, 3).double()
    d = pos[None, :, None, :] + (s @ cell)[None, None, :, :] - pos[:, None, None, :]
    r = d.norm(dim=-1)
    m = (r < cutoff) & (r > 1e-9)
    e = (torch.exp(-r) * m).sum()
    (g,) = torch.autograd.grad(e, pos)
    return e.detach(), -g


def test_aimnet2_adapter_pads_and_differentiates():
    batch = Batch.from_data_list([fcc_supercell(2, a=3.8, z=6, noise=0.1, seed=0, dtype=torch.float64)])
    w = AIMNet2Wrapper(_FakeAIMNet())
    w.model_config.active_outputs = {"energy", "forces", "stress", "charges", "node_embeddings"}
    _neighbors(w, batch)
    out = w(batch)
    e, f = _pair_reference(batch, 4.0)
    assert torch.allclose(out["energy"].reshape(()), e, atol=1e-10) and torch.allclose(out["forces"], f, atol=1e-10)
    assert out["charges"].shape == (batch.num_nodes,) and out["node_embeddings"].shape == (batch.num_nodes, 4)
    assert out["stress"].shape == (1, 3, 3) and not batch.positions.requires_grad
    assert w.distribution_spec().needs_total_charge


def test_uma_adapter_builds_edges_with_offsets():
    batch = Batch.from_data_list([fcc_supercell(2, a=3.8, z=6, noise=0.1, seed=1, dtype=torch.float64)])
    w = UMAWrapper(_FakeUMA(), cutoff=4.0)
    _neighbors(w, batch)
    out = w(batch)
    e, f = _pair_reference(batch, 4.0)
    assert torch.allclose(out["energy"].reshape(()), 0.5 * e, atol=1e-10)
    assert torch.allclose(out["forces"], 0.5 * f, atol=1e-10)
    assert w.distribution_spec().message_passes == 2
