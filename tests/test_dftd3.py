# SPDX-License-Identifier: Apache-2.0
"""DFT-D3(BJ): kernels against the differentiable PyTorch restatement, finite differences, parameter tables."""
from types import SimpleNamespace

import pytest
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch
from nvalchemi_toolkit_b200.models import dftd3 as d3
from nvalchemi_toolkit_b200.ops import _native


def _batch(seed=0, n=24, box=9.0):
    g = torch.Generator().manual_seed(seed)
    data = []
    for k in range(2):
        pos = torch.rand(n, 3, generator=g, dtype=torch.float64) * box
        z = torch.tensor([1, 6, 8, 14])[torch.randint(0, 4, (n,), generator=g)]
        data.append(AtomicData(atomic_numbers=z, positions=pos, cell=torch.eye(3, dtype=torch.float64) * box * (1 + 0.1 * k),
                               pbc=torch.tensor([True, True, True])))
    return Batch.from_data_list(data)


def _run(model, batch):
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    return model(batch)


def _model():
    m = d3.DFTD3ModelWrapper("pbe", parameters=d3.DFTD3Parameters.synthetic(20), cutoff=8.0, smoothing_width=1.5)
    m.model_config.active_outputs = {"energy", "forces", "stress", "virial", "atomic_energies", "coordination_numbers"}
    return m


def test_kernels_match_differentiable_restatement(monkeypatch):
    if not _native.available():
        pytest.skip("native library not built")
    model = _model()
    got = _run(model, _batch())
    monkeypatch.setattr(d3._native, "require", lambda t=None: False)
    want = _run(model, _batch())
    for k in ("energy", "forces", "virial", "atomic_energies", "coordination_numbers"):
        assert torch.allclose(got[k], want[k], rtol=1e-9, atol=1e-11), k
    assert float(got["energy"].abs().min()) > 1e-3 and float(got["forces"].abs().max()) > 1e-4


def test_forces_and_virial_match_finite_differences():
    model = _model()
    base = _batch(seed=2)
    out = _run(model, base)
    h = 1e-4

    def energy(mutate):
        b = _batch(seed=2)
        mutate(b)
        return _run(model, b)["energy"].reshape(-1)

    for i, c in ((0, 0), (7, 1), (30, 2)):
        def move(b, s):
            b.positions[i, c] += s * h
        fd = -(energy(lambda b: move(b, 1)) - energy(lambda b: move(b, -1))).sum() / (2 * h)
        assert abs(float(fd) - float(out["forces"][i, c])) < 1e-7

    def strain(b, s):
        eps = torch.zeros(3, 3, dtype=torch.float64)
        eps[0, 1] = eps[1, 0] = 0.5 * s * h
        eps[2, 2] = s * h
        d = torch.eye(3, dtype=torch.float64) + eps
        b["positions"] = b.positions @ d
        b["cell"] = b.cell.reshape(-1, 3, 3) @ d
    fd = (energy(lambda b: strain(b, 1)) - energy(lambda b: strain(b, -1))) / (2 * h)
    want = -(out["virial"][:, 0, 1] + out["virial"][:, 2, 2])
    assert torch.allclose(fd, want, atol=1e-6)


def test_energy_weights_select_owned_atoms():
    model = _model()
    b = _batch(seed=3)
    full = _run(model, b)
    b2 = _batch(seed=3)
    w = torch.zeros(b2.num_nodes, dtype=torch.float64)
    w[::2] = 1.0
    b2.add_key("energy_weights", w, level="node")
    part = _run(model, b2)
    e_want = torch.zeros(2, dtype=torch.float64).index_add_(0, b.batch_idx.long(), full["atomic_energies"] * w)
    assert torch.allclose(part["energy"].reshape(-1), e_want, atol=1e-12)
    b3 = _batch(seed=3)
    b3.add_key("energy_weights", 1.0 - w, level="node")
    rest = _run(model, b3)
    assert torch.allclose(part["forces"] + rest["forces"], full["forces"], atol=1e-12)  # the two halves add up


def test_parameter_tables_roundtrip_and_reference_table_parser(tmp_path):
    p = d3.DFTD3Parameters.synthetic(10)
    p.save(tmp_path / "d3.pt")
    q = d3.DFTD3Parameters.load(tmp_path / "d3.pt")
    assert torch.equal(p.c6ref, q.c6ref) and torch.equal(p.cnref, q.cnref)
    table = torch.tensor([[3.0, 1.0, 1.0, 0.9, 0.9], [7.5, 1.0, 6.0, 0.9, 0.0], [9.0, 1.0, 106.0, 0.9, 1.0],
                          [40.0, 106.0, 106.0, 1.0, 1.0]])
    r = d3.DFTD3Parameters.from_reference_table(table, torch.ones(7), torch.ones(7), max_z=6)
    assert r.c6ref[1, 1, 0, 0] == 3.0 and r.c6ref[6, 1, 0, 0] == 7.5 and r.c6ref[1, 6, 0, 1] == 9.0
    assert r.c6ref[6, 6, 1, 1] == 40.0 and r.cnref[6, 1] == 1.0 and r.c6ref[6, 6, 0, 0] == -1.0
    with pytest.raises(ValueError):
        d3.DFTD3ModelWrapper("pbe")
    assert d3.BJ_PARAMETERS["b3lyp"] == (1.0, 1.9889, 0.3981, 4.4211)
