# SPDX-License-Identifier: Apache-2.0
"""Classical models: Lennard-Jones kernel against an autograd restatement; thermostats and barostats driven by it."""
import pytest
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper, _lj_torch
from nvalchemi_toolkit_b200.neighbors import cell_and_pbc, compute_neighbors
from tests.helpers import fcc_supercell


def _lj_batch(device="cpu", dtype=torch.float32, cells=3, a=5.3):
    d1 = fcc_supercell(cells, a=a, z=18, noise=0.1, dtype=dtype)
    d2 = fcc_supercell(2, a=a * 1.02, z=18, noise=0.1, seed=4, dtype=dtype)
    return Batch.from_data_list([d1, d2], device=device)


@pytest.mark.parametrize("half", [False, True])
def test_lj_matches_autograd(device, half):
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0, half_list=half)
    model.model_config.active_outputs = {"energy", "forces", "stress"}
    b = _lj_batch(device)
    compute_neighbors(b, config=model.model_config.neighbor_config)
    out = model(b)
    cell, _ = cell_and_pbc(b)
    e_ref, f_ref, w_ref = _lj_torch(b.positions, cell, b.neighbor_matrix, b.neighbor_matrix_shifts, b.num_neighbors,
                                    b.batch_idx, 0.0104, 3.4, 8.0, 1.0, half, 2)
    e_sys = torch.zeros(2, dtype=e_ref.dtype, device=device).index_add_(0, b.batch_idx.long(), e_ref)
    assert torch.allclose(out["energy"].reshape(-1), e_sys, rtol=1e-4, atol=1e-5)
    assert torch.allclose(out["forces"], f_ref, rtol=1e-3, atol=1e-5)
    vol = torch.linalg.det(cell).abs()
    assert torch.allclose(out["stress"], -w_ref.reshape(2, 3, 3) / vol[:, None, None], rtol=1e-3, atol=1e-7)
    assert float(out["forces"].sum(0).abs().max()) < 1e-4


def _prime(dyn, b):
    from nvalchemi_toolkit_b200.dynamics import DynamicsStage

    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, b)
    dyn.compute(b)


def test_nose_hoover_holds_temperature():
    from nvalchemi_toolkit_b200.dynamics.integrators.nvt_nose_hoover import NVTNoseHoover

    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
    b = _lj_batch(dtype=torch.float64)
    _ops.initialize_velocities(b.velocities, b.atomic_masses, 60.0, b.batch_idx, random_seed=3)
    dyn = NVTNoseHoover(model, dt=2.0, temperature=60.0, thermostat_time=50.0, hooks=model.make_neighbor_hooks())
    _prime(dyn, b)
    temps = []
    for _ in range(150):
        dyn.step(b)
        ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, 2)
        temps.append(_ops.compute_temperature(ke, b.num_nodes_per_graph))
    t = torch.stack(temps[50:]).mean(0)
    assert (t > 35).all() and (t < 85).all()


def test_npt_relaxes_volume_towards_target_pressure():
    from nvalchemi_toolkit_b200.dynamics.integrators.npt import NPH, NPT

    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
    b = _lj_batch(dtype=torch.float64, a=5.0)  # compressed argon: positive pressure, cell must expand
    _ops.initialize_velocities(b.velocities, b.atomic_masses, 40.0, b.batch_idx, random_seed=3)
    v0 = torch.linalg.det(b.cell).abs().clone()
    dyn = NPT(model, dt=2.0, temperature=40.0, pressure=0.0, barostat_time=200.0, thermostat_time=50.0,
              hooks=model.make_neighbor_hooks())
    _prime(dyn, b)
    dyn.run(b, 120)
    v1 = torch.linalg.det(b.cell).abs()
    assert (v1 > v0 * 1.01).all() and torch.isfinite(b.positions).all()
    nph = NPH(model, dt=2.0, pressure=0.0, barostat_time=200.0, hooks=model.make_neighbor_hooks())
    _prime(nph, b)
    nph.run(b, 10)
    assert torch.isfinite(b.cell).all()


def test_fire2_and_variable_cell_relaxation():
    from nvalchemi_toolkit_b200.dynamics import ConvergenceHook
    from nvalchemi_toolkit_b200.dynamics.optimizers.fire2 import FIRE2
    from nvalchemi_toolkit_b200.dynamics.optimizers.fire_cell import FIREVariableCell

    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
    b = _lj_batch(dtype=torch.float64)
    opt = FIRE2(model, dt=0.05, tmax=0.5, convergence_hook=ConvergenceHook.from_fmax(1e-4), hooks=model.make_neighbor_hooks())
    _prime(opt, b)
    f0 = float(b.forces.norm(dim=-1).max())
    opt.run(b, 120)
    assert float(b.forces.norm(dim=-1).max()) < 0.3 * f0
    b2 = _lj_batch(dtype=torch.float64, a=5.0)
    vc = FIREVariableCell(model, dt=0.5, hooks=model.make_neighbor_hooks())
    _prime(vc, b2)
    p0 = -torch.diagonal(b2.stress, dim1=1, dim2=2).mean(-1)
    vc.run(b2, 60)
    p1 = -torch.diagonal(b2.stress, dim1=1, dim2=2).mean(-1)
    assert (p1.abs() < 0.5 * p0.abs()).all()


def test_triclinic_npt_relaxes_shear_without_rotating_the_cell():
    """Full 3 x 3 cell coupling: a sheared argon crystal under NPT(triclinic) loses its shear stress (the isotropic and
    per-axis modes cannot: their strain rate has no off-diagonal part), and the symmetric strain rate adds no rotation."""
    from nvalchemi_toolkit_b200.dynamics.integrators.npt import NPT

    def sheared():
        b = _lj_batch(dtype=torch.float64, a=5.3)
        shear = torch.eye(3, dtype=torch.float64)
        shear[0, 1] = shear[1, 0] = 0.03  # symmetric (pure) shear strain
        b["positions"] = b.positions @ shear
        cell = b.cell.reshape(-1, 3, 3)
        cell.copy_(cell @ shear)
        _ops.initialize_velocities(b.velocities, b.atomic_masses, 20.0, b.batch_idx, random_seed=5)
        return b

    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0, switch_width=1.0)
    res = {}
    for mode in ("triclinic", "anisotropic"):
        b = sheared()
        cell0 = b.cell.reshape(-1, 3, 3).clone()
        dyn = NPT(model, dt=2.0, temperature=20.0, pressure=0.0, barostat_time=150.0, thermostat_time=50.0,
                  pressure_coupling=mode, hooks=model.make_neighbor_hooks())
        _prime(dyn, b)
        s0 = b.stress.reshape(-1, 3, 3)[:, 0, 1].abs().clone()
        dyn.run(b, 150)
        cell1 = b.cell.reshape(-1, 3, 3)
        F = torch.linalg.solve(cell0, cell1)  # deformation gradient of the lattice (row convention)
        res[mode] = (s0, b.stress.reshape(-1, 3, 3)[:, 0, 1].abs(), (F - F.transpose(-1, -2)).abs().max(),
                     (cell1[:, 0] * cell1[:, 1]).sum(-1).abs())
        assert torch.isfinite(b.positions).all() and torch.isfinite(cell1).all()
    s0, s1, rot, _ = res["triclinic"]
    assert (s1 < 0.5 * s0).all(), (s0, s1)
    assert float(rot) < 5e-3          # symmetric strain rates: only the commutator of successive strains can rotate
    s0a, s1a, _, _ = res["anisotropic"]
    assert (s1a > 0.5 * s0a).all()    # the per-axis barostat cannot remove the shear


def test_nhc_and_barostat_kernels_match_torch_statements(device):
    """The chain kernel, the kinetic tensor and the per-system affine map against independent PyTorch expressions."""
    from nvalchemi_toolkit_b200.ops import _native

    if not _native.available():
        pytest.skip("native library not built")
    g = torch.Generator().manual_seed(0)
    m, c, n = 5, 3, 400
    b = torch.sort(torch.randint(0, m, (n,), generator=g)).values.to(torch.int32).to(device)
    v = torch.randn(n, 3, generator=g, dtype=torch.float64).to(device)
    f = torch.randn(n, 3, generator=g, dtype=torch.float64).to(device)
    mass = (torch.rand(n, generator=g, dtype=torch.float64) * 30 + 1).to(device)
    kt = _ops.compute_kinetic_tensor(v, mass, b, m)
    want = torch.zeros(m, 3, 3, dtype=torch.float64, device=device).index_add_(
        0, b.long(), mass[:, None, None] * v[:, :, None] * v[:, None, :])
    assert torch.allclose(kt, want, rtol=1e-12, atol=1e-12)
    # chain: kernel against the tensor-op statement, all Yoshida orders
    for order in (1, 3, 5):
        st = lambda: (torch.rand(m, generator=torch.Generator().manual_seed(order), dtype=torch.float64) * 4 + 1).to(device)  # noqa: E731
        ke2a, ke2b = st(), st()
        eta = [torch.zeros(m, c, dtype=torch.float64, device=device) for _ in range(2)]
        etd = [(torch.ones(m, c, dtype=torch.float64, device=device) * 0.01) for _ in range(2)]
        ndof = torch.full((m,), 30.0, dtype=torch.float64, device=device)
        kT = torch.full((m,), 0.02, dtype=torch.float64, device=device)
        dt = torch.full((m,), 0.3, dtype=torch.float64, device=device)
        Q = _ops.nhc_compute_masses(ndof, kT, torch.full_like(kT, 5.0), c)
        s_kernel = _ops.nhc_chain_scalar(ke2a, eta[0], etd[0], Q, kT, ndof, dt, order)
        s_torch = _ops._nhc_chain_torch(ke2b, eta[1], etd[1], Q, kT, ndof, dt, order)
        assert torch.allclose(s_kernel, s_torch, rtol=1e-12) and torch.allclose(ke2a, ke2b, rtol=1e-12)
        assert torch.allclose(eta[0], eta[1], rtol=1e-12, atol=1e-15) and torch.allclose(etd[0], etd[1], rtol=1e-12)
    # affine map with a kick before / after
    A = torch.randn(m, 3, 3, generator=g, dtype=torch.float64).to(device)
    C = torch.randn(m, 3, 3, generator=g, dtype=torch.float64).to(device)
    kick = (torch.rand(m, generator=g, dtype=torch.float64) + 0.1).to(device)
    for first in (False, True):
        x = v.clone()
        _ops.affine_rows_(x, A, b, y=f, C=C, forces=f, masses=mass, kick=kick, kick_first=first)
        k = (kick[b.long()] / mass).unsqueeze(-1) * f
        base = (v + k) if first else v
        want = torch.einsum("ip,ipq->iq", base, A[b.long()]) + torch.einsum("ip,ipq->iq", f, C[b.long()]) + (0 if first else k)
        assert torch.allclose(x, want, rtol=1e-12, atol=1e-12)


def test_fire2_kernel_matches_tensor_expressions(device, monkeypatch):
    """The four-phase FIRE2 kernel against the plain tensor statement of the same iteration, several steps in a row
    (downhill, uphill and step-capped systems), with and without the reduction seams a domain decomposition installs."""
    import nvalchemi_toolkit_b200.dynamics.optimizers.fire2 as f2

    if not f2._native.available():
        pytest.skip("native library not built")
    g = torch.Generator().manual_seed(3)
    sizes = [5, 9, 3, 7]
    n, m = sum(sizes), len(sizes)
    bidx = torch.repeat_interleave(torch.arange(m, dtype=torch.int32), torch.tensor(sizes)).to(device)
    hp = dict(delaystep=1, dtgrow=1.05, dtshrink=0.75, alphashrink=0.985, alpha0=0.09, tmax=0.08, tmin=0.005, maxstep=0.02)

    def run(kernel: bool, seams: bool):
        gg = torch.Generator().manual_seed(5)
        pos = torch.randn(n, 3, generator=gg, dtype=torch.float64).to(device)
        vel = (0.3 * torch.randn(n, 3, generator=gg, dtype=torch.float64)).to(device)
        alpha = torch.full((m,), 0.09, dtype=torch.float64, device=device)
        dt = torch.full((m,), 0.05, dtype=torch.float64, device=device)
        nsi = torch.zeros(m, dtype=torch.int32, device=device)
        calls = []
        red = (lambda t: (calls.append("sum"), t)[1]) if seams else None
        redmax = (lambda t: (calls.append("max"), t)[1]) if seams else None
        with monkeypatch.context() as mp:
            if not kernel:
                mp.setattr(f2._native, "available", lambda: False)
            for it in range(6):
                frc = torch.randn(n, 3, generator=gg, dtype=torch.float64).to(device) * (2.0 if it % 2 else 0.5)
                f2.fire2_step_coord(pos, vel, frc, bidx, alpha, dt, nsi, reduce=red, reduce_max=redmax, **hp)
        return pos.cpu(), vel.cpu(), alpha.cpu(), dt.cpu(), nsi.cpu(), calls

    want = run(False, False)
    for seams in (False, True):
        got = run(True, seams)
        for a, b in zip(got[:5], want[:5]):  # the step cap is reduced in float32: positions agree to ~1e-8 relative
            assert torch.allclose(a.double(), b.double(), rtol=1e-8, atol=1e-9)
        if seams:
            assert got[5][:4] == ["sum", "sum", "sum", "max"]


def test_functional_npt_ops():
    """The exported pieces of the MTK integrators: pressure tensor, scalar pressure, barostat mass, projection on the coupling
    mode, barostat half step, position / cell update (volume follows exp(dt tr v_g)), cell force of a hydrostatic stress."""
    from nvalchemi_toolkit_b200.dynamics import _ops

    torch.manual_seed(0)
    m = 2
    K = torch.randn(m, 3, 3, dtype=torch.float64)
    K = K @ K.transpose(1, 2)
    sigma = 0.01 * torch.randn(m, 3, 3, dtype=torch.float64)
    vol = torch.tensor([100.0, 250.0], dtype=torch.float64)
    P = _ops.compute_pressure_tensor(K, sigma, vol)
    assert torch.allclose(P, K / vol[:, None, None] - sigma)
    assert torch.allclose(_ops.compute_scalar_pressure(P), torch.stack([p.trace() / 3 for p in P]))
    ndof, kT, tau = torch.tensor([30.0, 60.0], dtype=torch.float64), torch.tensor([0.02, 0.03], dtype=torch.float64), torch.tensor([5.0, 7.0], dtype=torch.float64)
    W = _ops.compute_barostat_mass(ndof, kT, tau)
    assert torch.allclose(W, (ndof + 3) * kT * tau ** 2)
    g = torch.randn(m, 3, 3, dtype=torch.float64)
    iso, ani, tri = (_ops.project_cell_force(g, c) for c in ("isotropic", "anisotropic", "triclinic"))
    assert torch.allclose(iso, torch.diag_embed(torch.diagonal(g, dim1=1, dim2=2).mean(-1, keepdim=True).expand(-1, 3)))
    assert torch.allclose(ani, torch.diag_embed(torch.diagonal(g, dim1=1, dim2=2))) and torch.allclose(tri, tri.transpose(1, 2))
    with pytest.raises(ValueError):
        _ops.project_cell_force(g, "cubic")
    v_g = torch.zeros(m, 3, 3, dtype=torch.float64)
    dt = torch.tensor([0.5, 0.5], dtype=torch.float64)
    p_ext = torch.tensor([0.0, 0.001], dtype=torch.float64)
    ke2 = torch.diagonal(K, dim1=1, dim2=2).sum(-1)
    _ops.npt_barostat_half_step(v_g, P, p_ext, vol, ke2, ndof, W, dt, "triclinic")
    eye = torch.eye(3, dtype=torch.float64)
    want = 0.5 * dt[:, None, None] * _ops.project_cell_force(vol[:, None, None] * (P - p_ext[:, None, None] * eye) + (ke2 / ndof)[:, None, None] * eye, "triclinic") / W[:, None, None]
    assert torch.allclose(v_g, want) and _ops.nph_barostat_half_step is _ops.npt_barostat_half_step
    n = 7
    bidx = torch.tensor([0, 0, 0, 1, 1, 1, 1], dtype=torch.int32)
    pos, vel = torch.randn(n, 3, dtype=torch.float64), torch.randn(n, 3, dtype=torch.float64)
    cell = torch.stack([torch.eye(3, dtype=torch.float64) * 5, torch.eye(3, dtype=torch.float64) * 6])
    v_g = 0.01 * torch.randn(m, 3, 3, dtype=torch.float64)
    p0, c0 = pos.clone(), cell.clone()
    grow = _ops.npt_position_update(pos, vel, v_g, dt, bidx)
    _ops.npt_cell_update(cell, grow)
    b = bidx.long()
    half = dt[:, None, None] * torch.linalg.matrix_exp(0.5 * dt[:, None, None] * v_g)
    assert torch.allclose(pos, torch.einsum("ni,nij->nj", p0, grow[b]) + torch.einsum("ni,nij->nj", vel, half[b]))
    ratio = torch.linalg.det(cell) / torch.linalg.det(c0)
    assert torch.allclose(ratio, torch.exp(dt * torch.diagonal(v_g, dim1=1, dim2=2).sum(-1)))
    f = _ops.stress_to_cell_force(c0, -0.002 * eye.expand(m, 3, 3), factor=2.0)   # compressive stress pushes the cell outwards
    assert torch.allclose(f, 0.002 * torch.linalg.det(c0)[:, None, None] * c0 / 2.0)
