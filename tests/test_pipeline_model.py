# SPDX-License-Identifier: Apache-2.0
"""PipelineModelWrapper: additive groups, wiring, shared autograd, neighbour sharing, save/load."""
from types import SimpleNamespace

import pytest
import torch
from torch import nn

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.hooks import NeighborListHook
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
from nvalchemi_toolkit_b200.models.pipeline import (PipelineGroup, PipelineModelWrapper, PipelineStep,
                                                    filter_neighbor_matrix)
from tests.helpers import fcc_supercell


def _batch(n=3):
    return Batch.from_data_list([fcc_supercell(n, a=5.26, z=18, noise=0.05, seed=1, dtype=torch.float64)])


def _lj(cutoff, eps=0.0104):
    m = LennardJonesModelWrapper(epsilon=eps, sigma=3.4, cutoff=cutoff, switch_width=1.0)
    m.model_config.active_outputs = {"energy", "forces", "stress"}
    return m


def _neighbors(model, batch):
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)


def test_additive_groups_and_neighbor_sharing():
    a, b = _lj(6.0), _lj(4.5, eps=0.02)
    pipe = a + b
    assert isinstance(pipe, PipelineModelWrapper) and len(pipe.groups) == 2
    assert len(pipe._sources) == 1 and pipe.model_config.neighbor_config.cutoff == 6.0  # 6.0 <= 1.5 * 4.5: shared
    batch = _batch()
    _neighbors(pipe, batch)
    out = pipe(batch)
    ref = {}
    for m in (_lj(6.0), _lj(4.5, eps=0.02)):
        bb = _batch()
        _neighbors(m, bb)
        o = m(bb)
        for k in ("energy", "forces", "stress"):
            ref[k] = o[k] if k not in ref else ref[k] + o[k]
    for k in ("energy", "forces", "stress"):
        assert torch.allclose(out[k], ref[k], atol=1e-10), k
    # far-apart cutoffs get their own lists under "auto", one list under "always"
    far = PipelineModelWrapper([PipelineGroup([_lj(9.0)]), PipelineGroup([_lj(4.0)])])
    assert len(far._sources) == 2
    one = PipelineModelWrapper([PipelineGroup([_lj(9.0)]), PipelineGroup([_lj(4.0)])], neighbor_adaptation="always")
    assert len(one._sources) == 1
    with pytest.raises(ValueError):
        PipelineModelWrapper([PipelineGroup([_lj(4.0)])], neighbor_adaptation="sometimes")


def test_filter_neighbor_matrix_matches_direct_build():
    from nvalchemi_toolkit_b200 import neighbors as nb

    batch = _batch()
    nb.compute_neighbors(batch, 6.0, max_neighbors=96)
    nm, num, sh = filter_neighbor_matrix(batch.positions, batch.cell.reshape(-1, 3, 3), batch.batch_idx,
                                         batch.neighbor_matrix, batch.num_neighbors, batch.neighbor_matrix_shifts, 4.5)
    b2 = _batch()
    nb.compute_neighbors(b2, 4.5, max_neighbors=96)
    assert torch.equal(num, b2.num_neighbors)
    for i in range(0, batch.num_nodes, 7):
        got = {(int(j), *map(int, s)) for j, s in zip(nm[i, : num[i]], sh[i, : num[i]])}
        want = {(int(j), *map(int, s)) for j, s in zip(b2.neighbor_matrix[i, : num[i]], b2.neighbor_matrix_shifts[i, : num[i]])}
        assert got == want


class _Charges(nn.Module, BaseModelMixin):
    """Position-dependent per-atom 'charges' and a small energy (differentiable)."""

    def __init__(self):
        super().__init__()
        self.w = nn.Parameter(torch.tensor([0.3, -0.2, 0.1], dtype=torch.float64))
        self.model_config = ModelConfig(outputs=frozenset({"energy", "charges"}), supports_pbc=True)

    def checkpoint_spec(self):
        return {"cls": "tests.test_pipeline_model._Charges", "config": {}}

    def forward(self, data, **kw):
        q = torch.sin(data.positions @ self.w)
        e = torch.zeros(data.num_graphs, 1, dtype=q.dtype).index_add_(0, data.batch_idx.long(), (0.1 * q * q)[:, None])
        return self.adapt_output({"energy": e, "charges": q}, data)


class _ChargeEnergy(nn.Module, BaseModelMixin):
    """Energy from wired charges: ``E = k * sum_i q_i^2 * |r_i|^2``."""

    def __init__(self, k=0.05):
        super().__init__()
        self.k = k
        self.model_config = ModelConfig(outputs=frozenset({"energy"}), required_inputs=frozenset({"node_charges"}),
                                        supports_pbc=True)

    def checkpoint_spec(self):
        return {"cls": "tests.test_pipeline_model._ChargeEnergy", "config": {"k": self.k}}

    def forward(self, data, **kw):
        q = data.node_charges
        e_atom = self.k * q * q * data.positions.pow(2).sum(-1)
        e = torch.zeros(data.num_graphs, 1, dtype=q.dtype).index_add_(0, data.batch_idx.long(), e_atom[:, None])
        return self.adapt_output({"energy": e}, data)


def test_wired_autograd_group_differentiates_through_the_wire():
    pipe = PipelineModelWrapper([PipelineGroup(steps=[PipelineStep(_Charges(), wire={"charges": "node_charges"}),
                                                      _ChargeEnergy()], use_autograd=True)])
    pipe.model_config.active_outputs = {"energy", "forces", "stress"}
    assert "node_charges" not in pipe.model_config.required_inputs  # provided by the wire
    batch = _batch(2)
    out = pipe(batch)
    pos = batch.positions.clone().requires_grad_(True)
    w = pipe._models[0].w.detach()
    q = torch.sin(pos @ w)
    e = (0.1 * q * q).sum() + (0.05 * q * q * pos.pow(2).sum(-1)).sum()
    (g,) = torch.autograd.grad(e, pos)
    assert torch.allclose(out["energy"].reshape(()), e.detach(), atol=1e-10)
    assert torch.allclose(out["forces"], -g, atol=1e-10)
    # stress from the strain trick equals sum_i r_i (x) dE/dr_i / V for this cell-independent energy
    vol = torch.linalg.det(batch.cell.reshape(3, 3))
    want = torch.einsum("ni,nj->ij", pos.detach(), g) / vol
    assert torch.allclose(out["stress"].reshape(3, 3), 0.5 * (want + want.t()), atol=1e-10)
    assert not batch.positions.requires_grad and torch.equal(batch.positions, pos.detach())
    # a missing wire is reported at construction
    with pytest.raises(ValueError):
        PipelineModelWrapper([PipelineGroup(steps=[PipelineStep(_Charges(), wire={"dipole": "node_charges"})])])
    lonely = PipelineModelWrapper([PipelineGroup(steps=[_ChargeEnergy()])])
    assert "node_charges" in lonely.model_config.required_inputs


def test_custom_derivative_fn_and_mixed_groups():
    seen = {}

    def deriv(energy, data, requested):
        seen["requested"] = set(requested)
        leaf = data._pipeline_leaves["positions"]
        (g,) = torch.autograd.grad(energy.sum(), leaf)
        return {"forces": -2.0 * g}

    auto = PipelineGroup(steps=[PipelineStep(_Charges(), wire={"charges": "node_charges"}), _ChargeEnergy()],
                         use_autograd=True, derivative_fn=deriv)
    pipe = PipelineModelWrapper([auto, PipelineGroup(steps=[_lj(6.0)])])
    pipe.model_config.active_outputs = {"energy", "forces"}
    batch = _batch(3)
    _neighbors(pipe, batch)
    out = pipe(batch)
    assert seen["requested"] == {"forces"}
    plain = PipelineModelWrapper([PipelineGroup(steps=[PipelineStep(_Charges(), wire={"charges": "node_charges"}),
                                                       _ChargeEnergy()], use_autograd=True)])
    plain.model_config.active_outputs = {"energy", "forces"}
    f_auto = plain(_batch(3))["forces"]
    b2 = _batch(3)
    lj = _lj(6.0)
    _neighbors(lj, b2)
    f_lj = lj(b2)["forces"]
    assert torch.allclose(out["forces"], 2.0 * f_auto + f_lj, atol=1e-10)


def test_pipeline_save_load_roundtrip(tmp_path):
    pipe = PipelineModelWrapper([PipelineGroup(steps=[PipelineStep(_Charges(), wire={"charges": "node_charges"}),
                                                      _ChargeEnergy(0.07)], use_autograd=True),
                                 PipelineGroup(steps=[_lj(6.0)])])
    with torch.no_grad():
        pipe._models[0].w.mul_(1.5)
    pipe.model_config.active_outputs = {"energy", "forces"}
    path = tmp_path / "pipe.pt"
    pipe.save(path)
    again = PipelineModelWrapper.load(path)
    b1, b2 = _batch(3), _batch(3)
    _neighbors(pipe, b1)
    _neighbors(again, b2)
    o1, o2 = pipe(b1), again(b2)
    assert torch.allclose(o1["energy"], o2["energy"]) and torch.allclose(o1["forces"], o2["forces"])
    assert again.groups[0].use_autograd and again.groups[0].steps[0].wire == {"charges": "node_charges"}
