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
