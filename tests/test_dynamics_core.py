# SPDX-License-Identifier: Apache-2.0
"""Step loop, hooks, convergence, stage fusion and integrator physics on the demo model."""
import pytest
import torch

from nvalchemi_toolkit_b200.dynamics import (FIRE, NVE, ConvergenceHook, DemoDynamics, DynamicsStage, FusedStage,
                                             NVTLangevin, _ops)
from nvalchemi_toolkit_b200.models import DemoModelWrapper
from tests.helpers import random_batch


class RecordingHook:
    def __init__(self, stage, frequency=1):
        self.stage, self.frequency, self.calls = stage, frequency, []

    def __call__(self, ctx, stage):
        self.calls.append((ctx.step_count, stage))


def test_stage_order_and_frequency():
    b = random_batch([4, 6])
    hooks = [RecordingHook(s) for s in DynamicsStage if s != DynamicsStage.ON_CONVERGE]
    every2 = RecordingHook(DynamicsStage.AFTER_STEP, frequency=2)
    dyn = DemoDynamics(DemoModelWrapper(), n_steps=4, dt=0.01, hooks=hooks + [every2])
    dyn.run(b)
    assert all(len(h.calls) == 4 for h in hooks)
    assert [c[0] for c in every2.calls] == [0, 2]
    with pytest.raises(ValueError):
        dyn.register_hook(RecordingHook(DynamicsStage.AFTER_STEP, frequency=0))

    class Other:
        frequency, stage = 1, None

        def __call__(self, ctx, stage):
            pass

    with pytest.raises(TypeError):
        dyn.register_hook(Other())


def test_nve_energy_conservation(device):
    torch.manual_seed(0)
    b = random_batch([int(n) for n in torch.randint(8, 33, (16,))], device=device)
    _ops.initialize_velocities(b.velocities, b.atomic_masses, 300.0, b.batch_idx, random_seed=0)
    model = DemoModelWrapper().to(device)
    dyn = NVE(model, dt=0.5)
    dyn.compute(b)
    ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs)
    e0 = b.energy.squeeze(-1) + ke
    dyn.run(b, 100)
    ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs)
    drift = ((b.energy.squeeze(-1) + ke) - e0).abs().max()
    assert float(drift) < 5e-3
    assert dyn.step_count == 100 and not b.positions.requires_grad


def test_langevin_thermalises(device):
    b = random_batch([32] * 8, device=device)

    class Zero(DemoModelWrapper):
        def forward(self, data, **kw):
            return {"energy": torch.zeros(data.num_graphs, 1, device=data.device), "forces": torch.zeros_like(data.positions)}

    dyn = NVTLangevin(Zero().to(device), dt=1.0, temperature=300.0, friction=0.1, random_seed=1)
    b["forces"] = torch.zeros_like(b.positions)
    dyn.run(b, 300)
    ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs)
    t = _ops.compute_temperature(ke, b.num_nodes_per_graph).mean()
    assert 240 < float(t) < 360


def test_fire_reduces_forces_and_converges():
    b = random_batch([10, 12])
    model = DemoModelWrapper()
    probe = FIRE(model, dt=0.1)
    probe.compute(b)
    f0 = float(b.forces.norm(dim=-1).max())
    dyn = FIRE(model, dt=0.5, convergence_hook=ConvergenceHook.from_fmax(0.5 * f0))
    dyn.run(b, 2000)
    assert float(b.forces.norm(dim=-1).max()) <= 0.5 * f0 + 1e-7
    assert dyn.step_count < 2000


def test_frozen_systems_do_not_move():
    b = random_batch([5, 5])
    b.add_key("status", torch.tensor([[0], [1]]), level="system")
    p1 = b.positions[5:].clone()
    dyn = DemoDynamics(DemoModelWrapper(), n_steps=3, dt=0.05)
    dyn.compute(b)
    dyn.run(b)
    assert torch.equal(b.positions[5:], p1) and not torch.equal(b.positions[:5], b.positions[:5] * 0 + p1[:5])


def test_fused_stage_migrates_status():
    b = random_batch([6, 6, 6])
    model = DemoModelWrapper()
    relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(1e9))  # converges at once
    md = NVE(model, dt=0.5, n_steps=3)
    fused = relax + md
    assert isinstance(fused, FusedStage) and fused.exit_status == 2
    out = fused.run(b, n_steps=10)
    assert out.status.reshape(-1).tolist() == [2, 2, 2]
    assert fused.step_count == 3  # the migration step already counts toward the MD budget (as in the reference)


def test_reference_operator_names_are_callable():
    """Call sites written against ``torch.ops.nvalchemi.*`` / ``torch.ops.nvalchemi_hooks.*`` keep working."""
    import torch

    import nvalchemi_toolkit_b200  # noqa: F401  (registers the operators)
    from nvalchemi_toolkit_b200.ops import compat

    assert {"initialize_velocities", "velocity_rescale", "remove_com_motion", "compute_temperature", "align_cell",
            "lj_energy_forces_batch", "per_system_reduce", "segmented_sum", "wrap_positions"} <= set(compat.registered_names())
    n, m = 12, 3
    vel = torch.zeros(n, 3, dtype=torch.float64)
    masses = torch.full((n,), 12.0, dtype=torch.float64)
    batch_idx = torch.arange(m, dtype=torch.int32).repeat_interleave(4)
    torch.ops.nvalchemi.initialize_velocities(vel, masses, torch.full((m,), 300.0, dtype=torch.float64), batch_idx, 7)
    ke = torch.ops.nvalchemi_hooks.compute_kinetic_energy(vel, masses, batch_idx, m)
    temp = torch.ops.nvalchemi.compute_temperature(ke, torch.full((m,), 4))
    assert torch.allclose(temp, torch.full((m,), 300.0, dtype=torch.float64), rtol=1e-6)
    torch.ops.nvalchemi.velocity_rescale(vel, torch.full((m,), 2.0, dtype=torch.float64), batch_idx)
    assert torch.allclose(torch.ops.nvalchemi_hooks.compute_kinetic_energy(vel, masses, batch_idx, m), 4 * ke)
    s = torch.ops.nvalchemi_hooks.segmented_sum(torch.ones(n, 2, dtype=torch.float64), batch_idx, m)
    assert torch.equal(s, torch.full((m, 2), 4.0, dtype=torch.float64))
    assert torch.equal(torch.ops.nvalchemi.per_system_reduce(torch.ones(n, dtype=torch.float64), batch_idx, m),
                       torch.full((m,), 4.0, dtype=torch.float64))


def test_neighbor_hook_methods_agree_and_width_shrinks():
    """``method="naive"`` and the cell list give the same neighbour sets; a matrix much wider than needed shrinks after a
    few rebuilds; unknown methods and the accepted-but-ineffective ``compile`` switches say so."""
    import warnings
    from types import SimpleNamespace

    import pytest
    import torch

    from nvalchemi_toolkit_b200 import Batch
    from nvalchemi_toolkit_b200.distributed import DomainConfig
    from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook
    from nvalchemi_toolkit_b200.models.base import NeighborConfig, NeighborListFormat
    from tests.helpers import fcc_supercell

    cfg = NeighborConfig(cutoff=4.0, format=NeighborListFormat.MATRIX)
    sets = {}
    for method in ("cell_list", "naive"):
        b = Batch.from_data_list([fcc_supercell(2, noise=0.05, seed=1, dtype=torch.float64)])
        h = NeighborListHook(cfg, method=method)
        h(SimpleNamespace(batch=b), None)
        nm, num = b.neighbor_matrix, b.num_neighbors
        sets[method] = [sorted(nm[i, : int(num[i])].tolist()) for i in range(b.num_nodes)]
    assert sets["cell_list"] == sets["naive"]
    with pytest.raises(ValueError):
        NeighborListHook(cfg, method="octree")
    b = Batch.from_data_list([fcc_supercell(2, noise=0.05, seed=1, dtype=torch.float64)])
    h = NeighborListHook(cfg)
    h.shrink_after = 2
    h(SimpleNamespace(batch=b), None)
    h._alloc(b, 512)  # pretend an earlier, denser state had widened the matrix
    for _ in range(3):
        h(SimpleNamespace(batch=b), None)
    assert b.neighbor_matrix.shape[1] < 512 and int(b.num_neighbors.max()) <= b.neighbor_matrix.shape[1]
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        DomainConfig(cutoff=5.0, compile=True)
    assert any("no effect" in str(x.message) for x in w)


def test_native_integrator_ops_trace_as_opaque_nodes():
    """A velocity-Verlet step written with the native operators traces under ``torch.compile(fullgraph=True)`` (the
    operators carry fake implementations) and gives the eager result."""
    import pytest
    import torch

    from nvalchemi_toolkit_b200.ops import _native

    if not _native.available():
        pytest.skip("native library not built")
    import nvalchemi_toolkit_b200.ops.compat  # noqa: F401  (registers the fake implementations)

    def step(pos, vel, frc, mass, dt, b):
        torch.ops.nvalchemi.vv_position_update(pos, vel, frc, mass, dt, b)
        torch.ops.nvalchemi.vv_velocity_finalize(vel, frc, mass, dt, b)
        return torch.ops.nvalchemi.compute_kinetic_energy(vel, mass, b, 2)

    def state():
        g = torch.Generator().manual_seed(0)
        return (torch.randn(10, 3, generator=g), torch.randn(10, 3, generator=g), torch.randn(10, 3, generator=g),
                torch.rand(10, generator=g) + 1.0, torch.tensor([0.5, 0.25]), torch.tensor([0] * 6 + [1] * 4, dtype=torch.int32))

    a, b = state(), state()
    ke_eager = step(*a)
    ke_traced = torch.compile(step, fullgraph=True, backend="eager")(*b)
    assert torch.allclose(ke_eager, ke_traced) and torch.allclose(a[0], b[0]) and torch.allclose(a[1], b[1])
