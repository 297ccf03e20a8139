# SPDX-License-Identifier: Apache-2.0
"""Ewald and PME: Madelung constant, analytic forces / virial / potentials against finite differences, kernel pieces
against their PyTorch restatements, differentiability with respect to charges."""
import math
from types import SimpleNamespace

import pytest
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch
from nvalchemi_toolkit_b200.models import _electrostatics as es
from nvalchemi_toolkit_b200.models.ewald import EwaldModelWrapper
from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper


def _nacl(n=2, a=5.64, noise=0.0, seed=0, charge_noise=0.0):
    g = torch.Generator().manual_seed(seed)
    r = torch.arange(2 * n, dtype=torch.float64)
    grid = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3)
    pos = grid * (a / 2) + noise * torch.randn(grid.shape, generator=g, dtype=torch.float64)
    q = torch.where(grid.sum(-1) % 2 == 0, 1.0, -1.0).double()
    q = q + charge_noise * torch.randn(q.shape, generator=g, dtype=torch.float64)
    z = torch.where(q > 0, 11, 17)
    d = AtomicData(atomic_numbers=z, positions=pos, cell=torch.eye(3, dtype=torch.float64) * a * n,
                   pbc=torch.tensor([True, True, True]))
    b = Batch.from_data_list([d])
    b.add_key("node_charges", q, level="node")
    return b


def _run(model, batch):
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    return model(batch)


@pytest.mark.parametrize("cls,tol", [(EwaldModelWrapper, 1e-6), (PMEModelWrapper, 2e-5)])
def test_madelung_constant_of_rock_salt(cls, tol):
    batch = _nacl(2)
    model = cls(cutoff=5.5, accuracy=1e-8)
    out = _run(model, batch)
    per_pair = float(out["energy"]) / (batch.num_nodes / 2)
    want = -1.7475645946 * es.COULOMB_EV_A / (5.64 / 2)
    assert abs(per_pair - want) < tol * abs(want)
    assert float(out["forces"].abs().max()) < 1e-6


@pytest.mark.parametrize("cls,ftol", [(EwaldModelWrapper, 1e-6), (PMEModelWrapper, 5e-5)])
def test_forces_virial_and_potentials_match_finite_differences(cls, ftol):
    model = cls(cutoff=5.5, accuracy=1e-8)
    model.model_config.active_outputs = {"energy", "forces", "stress", "virial", "electrostatic_potential"}
    base = _nacl(2, noise=0.15, seed=1, charge_noise=0.05)  # net charge != 0: exercises the background term

    def energy(mutate):
        b = _nacl(2, noise=0.15, seed=1, charge_noise=0.05)
        mutate(b)
        model.invalidate_cache()
        return float(_run(model, b)["energy"])

    out = _run(model, base)
    h = 1e-4
    for i, c in ((0, 0), (5, 2), (17, 1)):
        def up(b, s=1.0):
            b.positions[i, c] += s * h
        fd = -(energy(lambda b: up(b, 1.0)) - energy(lambda b: up(b, -1.0))) / (2 * h)
        assert abs(fd - float(out["forces"][i, c])) < ftol * max(1.0, abs(fd)) * 20
    for i in (3, 11):
        def upq(b, s=1.0):
            b.node_charges[i] += s * h
        fd = (energy(lambda b: upq(b, 1.0)) - energy(lambda b: upq(b, -1.0))) / (2 * h)
        assert abs(fd - float(out["electrostatic_potential"][i])) < 20 * ftol * max(1.0, abs(fd))
    for a, c in ((0, 0), (1, 2), (2, 2)):
        def strain(b, s=1.0):
            eps = torch.zeros(3, 3, dtype=torch.float64)
            eps[a, c] += 0.5 * s * h
            eps[c, a] += 0.5 * s * h
            d = torch.eye(3, dtype=torch.float64) + eps
            b["positions"] = b.positions @ d
            b["cell"] = (b.cell.reshape(3, 3) @ d).reshape(1, 3, 3)
        fd = (energy(lambda b: strain(b, 1.0)) - energy(lambda b: strain(b, -1.0))) / (2 * h)
        assert abs(-fd - float(out["virial"][0, a, c])) < 50 * ftol * max(1.0, abs(fd))
    vol = float(torch.linalg.det(base.cell.reshape(3, 3)))
    assert torch.allclose(out["stress"], -out["virial"] / vol)


def test_pme_agrees_with_ewald_and_kernels_with_torch_restatement():
    batch = _nacl(2, noise=0.2, seed=4)
    e = EwaldModelWrapper(cutoff=5.5, accuracy=1e-8)
    p = PMEModelWrapper(cutoff=5.5, accuracy=1e-8, spline_order=6)
    for m in (e, p):
        m.model_config.active_outputs = {"energy", "forces", "stress"}
    oe, op = _run(e, batch), _run(p, _nacl(2, noise=0.2, seed=4))
    assert abs(float(oe["energy"] - op["energy"])) < 1e-4 * abs(float(oe["energy"]))
    assert float((oe["forces"] - op["forces"]).abs().max()) < 2e-4
    assert float((oe["stress"] - op["stress"]).abs().max()) < 1e-5
    # mesh stages: OpenMP/CUDA functors against plain PyTorch
    pos, q = batch.positions, batch.node_charges
    cell = batch.cell.reshape(3, 3)
    inv = torch.linalg.inv(cell).contiguous()
    dims, order = (12, 15, 16), 5
    mod = tuple(es.bspline_moduli(n, order) for n in dims)
    want = es._spread_torch(pos, q, inv, dims, order, 0, pos.shape[0], None)
    got = torch.ops.nvalchemi.pme_spread(pos, q, inv, *dims, order, 0, pos.shape[0], None)
    assert torch.allclose(got, want, atol=1e-12)
    fk = torch.fft.rfftn(want)
    fk_t, e_t, w_t = es._convolve_torch(fk.clone(), inv, mod, 0.35, float(torch.linalg.det(cell)), dims)
    raw = torch.view_as_real(fk.clone()).contiguous()
    acc = torch.ops.nvalchemi.pme_convolve(raw, inv, *mod, 0.35, float(torch.linalg.det(cell)), dims[2])
    assert torch.allclose(torch.view_as_complex(raw), fk_t, atol=1e-10)
    assert abs(float(acc[0] - e_t)) < 1e-10 and torch.allclose(acc[[1, 2, 3, 4, 5, 6]], w_t[[0, 0, 0, 1, 1, 2], [0, 1, 2, 1, 2, 2]])
    phi_mesh = torch.fft.irfftn(fk_t, s=dims, norm="forward").contiguous()
    f_t, p_t = es._gather_torch(pos, q, inv, phi_mesh, dims, order, 0, pos.shape[0])
    f_k, p_k = torch.ops.nvalchemi.pme_gather(pos, q, inv, phi_mesh, order, 0, pos.shape[0])
    assert torch.allclose(f_k, f_t, atol=1e-10) and torch.allclose(p_k, p_t, atol=1e-10)
    # real space and structure factors
    nb = 1
    alpha = torch.tensor([0.35], dtype=torch.float64)
    args = (pos, q, batch.cell.reshape(1, 3, 3), batch.neighbor_matrix, batch.neighbor_matrix_shifts, batch.num_neighbors,
            batch.batch_idx, alpha, 5.5, False, nb)
    for a, b in zip(es.real_space(*args), es._real_space_torch(*args)):
        assert torch.allclose(a.reshape(b.shape), b, atol=1e-10)


def test_energy_is_differentiable_in_charges_positions_and_strain():
    batch = _nacl(2, noise=0.1, seed=2)
    model = EwaldModelWrapper(cutoff=5.5, accuracy=1e-8)
    model.model_config.active_outputs = {"energy", "forces", "virial", "electrostatic_potential"}
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    q = batch.node_charges.clone().requires_grad_(True)
    pos = batch.positions.clone().requires_grad_(True)
    strain = torch.zeros(3, 3, dtype=torch.float64, requires_grad=True)
    d = torch.eye(3, dtype=torch.float64) + 0.5 * (strain + strain.t())
    cell0 = batch.cell.reshape(3, 3).clone()
    batch["node_charges"], batch["positions"], batch["cell"] = q * 1.0, pos @ d, (cell0 @ d).reshape(1, 3, 3)
    out = model(batch)
    gq, gp, gs = torch.autograd.grad(out["energy"].sum(), [q, pos, strain])
    assert torch.allclose(gq, out["electrostatic_potential"], atol=1e-10)
    assert torch.allclose(gp, -out["forces"], atol=1e-10)
    assert torch.allclose(gs, -out["virial"][0], atol=1e-8)


def test_slab_correction_force_matches_finite_difference():
    model = EwaldModelWrapper(cutoff=5.5, accuracy=1e-8, slab_correction=True)
    plain = EwaldModelWrapper(cutoff=5.5, accuracy=1e-8)

    def energy(dz, m):
        b = _nacl(2, noise=0.1, seed=3)
        b.positions[7, 2] += dz
        return float(_run(m, b)["energy"])

    b = _nacl(2, noise=0.1, seed=3)
    out, ref = _run(model, b), _run(plain, _nacl(2, noise=0.1, seed=3))
    h = 1e-4
    fd = -(energy(h, model) - energy(-h, model)) / (2 * h)
    assert abs(fd - float(out["forces"][7, 2])) < 1e-5
    q, z = b.node_charges, b.positions[:, 2]
    vol = float(torch.linalg.det(b.cell.reshape(3, 3)))
    want = 2 * math.pi / vol * float((q * z).sum()) ** 2 * es.COULOMB_EV_A
    assert abs(float(out["energy"] - ref["energy"]) - want) < 1e-9
