# SPDX-License-Identifier: Apache-2.0
"""Stock hooks one by one: registration rules, bias potentials, force clamping, NaN detection, drift monitoring, frozen
atoms, periodic wrapping, converged snapshots."""
import warnings

import pytest
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch
from nvalchemi_toolkit_b200.dynamics import NVE, DynamicsStage, _ops
from nvalchemi_toolkit_b200.dynamics.hooks import (ConvergedSnapshotHook, EnergyDriftMonitorHook, FreezeAtomsHook,
                                                  MaxForceClampHook, NaNDetectorHook)
from nvalchemi_toolkit_b200.dynamics.sinks import HostMemory
from nvalchemi_toolkit_b200.hooks.bias import BiasedPotentialHook
from nvalchemi_toolkit_b200.hooks.periodic import WrapPeriodicHook
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper
from tests.helpers import random_batch


def _engine(hooks=(), dt=0.5, double=False):
    torch.manual_seed(0)  # every engine of a test evaluates the same network
    model = DemoModelWrapper().double() if double else DemoModelWrapper()
    return NVE(model, dt=dt, hooks=list(hooks))


def test_registration_rules():
    class NoStage:
        frequency = 1

        def __call__(self, ctx, stage):
            pass

    with pytest.raises(TypeError, match="no stage assigned"):
        _engine([NoStage()])
    eng = _engine()
    eng.register_hook(NoStage(), stage=DynamicsStage.AFTER_STEP)   # a stage given at registration is enough
    assert eng.hooks[-1].stage == DynamicsStage.AFTER_STEP

    class BadFrequency(NoStage):
        frequency = 0
        stage = DynamicsStage.AFTER_STEP

    with pytest.raises(ValueError, match="positive integer"):
        _engine([BadFrequency()])

    class WrongEnum(NoStage):
        from nvalchemi_toolkit_b200.training import TrainingStage

        stage = TrainingStage.AFTER_BACKWARD

    with pytest.raises(TypeError, match="only accepts"):
        _engine([WrongEnum()])
    # hooks shared between engines choose their default stage when they are registered
    wrap, bias = WrapPeriodicHook(), BiasedPotentialHook(lambda b: (None, None))
    eng = _engine([wrap, bias])
    assert wrap.stage == DynamicsStage.AFTER_POST_UPDATE and bias.stage == DynamicsStage.AFTER_COMPUTE


def test_hooks_fire_in_registration_order_at_their_frequency():
    calls = []

    class Probe:
        def __init__(self, name, frequency, stage):
            self.name, self.frequency, self.stage = name, frequency, stage

        def __call__(self, ctx, stage):
            calls.append((ctx.step_count, self.name))

    b = random_batch([4])
    eng = _engine([Probe("a", 1, DynamicsStage.AFTER_STEP), Probe("b", 2, DynamicsStage.AFTER_STEP),
                   Probe("c", 1, DynamicsStage.BEFORE_STEP)])
    eng.run(b, 4)
    after = [(s, n) for s, n in calls if n != "c"]
    steps_b = [s for s, n in after if n == "b"]
    assert len([1 for _, n in calls if n == "c"]) == 4 and len([1 for _, n in after if n == "a"]) == 4
    assert len(steps_b) == 2 and all(s % 2 == 0 for s in steps_b)
    for s in steps_b:  # on shared steps, "a" (registered first) precedes "b"
        assert after.index((s, "a")) < after.index((s, "b"))


@pytest.mark.parametrize("inplace", [True, False])
def test_bias_hook_adds_a_harmonic_restraint(inplace):
    b = random_batch([3, 5], dtype=torch.float64)
    centre = b.positions.mean(0, keepdim=True)

    def restraint(batch):
        d = batch.positions - centre
        e = torch.zeros(batch.num_graphs, dtype=d.dtype).index_add_(0, batch.batch_idx.long(), 0.5 * 0.3 * (d * d).sum(-1))
        return e, -0.3 * d

    plain = _engine(double=True)
    plain.compute(b)
    e0, f0 = b.energy.clone(), b.forces.clone()
    eng = _engine([BiasedPotentialHook(restraint, inplace=inplace)], double=True)
    eng.compute(b)
    eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    e_bias, f_bias = restraint(b)
    assert torch.allclose(b.energy.reshape(-1), e0.reshape(-1) + e_bias) and torch.allclose(b.forces, f0 + f_bias)
    # energy-only and force-only biases are both allowed
    eng2 = _engine([BiasedPotentialHook(lambda batch: (torch.ones(batch.num_graphs, dtype=torch.float64), None))], double=True)
    eng2.compute(b)
    before = b.forces.clone()
    eng2._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    assert torch.equal(b.forces, before)


def test_force_clamp_preserves_direction_and_small_forces():
    with pytest.raises(ValueError):
        MaxForceClampHook(0.0)
    b = random_batch([6])
    eng = _engine([MaxForceClampHook(2.0)])
    eng.compute(b)
    f = torch.tensor([[3.0, 4.0, 0.0], [0.1, 0.0, 0.0], [0.0, 0.0, -10.0], [0.0, 0.0, 0.0], [1.0, 1.0, 1.0], [2.0, 0.0, 0.0]])
    b.forces.copy_(f)
    eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    out = b.forces
    assert torch.allclose(out[0], torch.tensor([1.2, 1.6, 0.0])) and torch.allclose(out[2], torch.tensor([0.0, 0.0, -2.0]))
    assert torch.equal(out[1], f[1]) and torch.equal(out[3], f[3]) and torch.equal(out[4], f[4]) and torch.equal(out[5], f[5])
    assert float(out.norm(dim=-1).max()) <= 2.0 + 1e-6


def test_nan_detector_names_the_graphs_and_checks_extra_keys():
    b = random_batch([3, 4, 2])
    eng = _engine([NaNDetectorHook(extra_keys=["velocities"])])
    eng.compute(b)
    eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)          # clean batch: silent
    b.forces[4, 1] = float("inf")                             # atom 4 lives in graph 1
    with pytest.raises(RuntimeError, match=r"'forces'.*graphs \[1\]"):
        eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    b.forces[4, 1] = 0.0
    b.velocities[8, 0] = float("nan")                         # graph 2, only seen through extra_keys
    with pytest.raises(RuntimeError, match=r"'velocities'.*graphs \[2\]"):
        eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    b.velocities[8, 0] = 0.0
    b.energy[0] = float("nan")
    with pytest.raises(RuntimeError, match=r"'energy'.*graphs \[0\]"):
        eng._call_hooks(DynamicsStage.AFTER_COMPUTE, b)


def test_energy_drift_monitor_metrics_and_actions():
    b = random_batch([4, 4], dtype=torch.float64)
    mon = EnergyDriftMonitorHook(1e-3, metric="absolute", action="raise", include_kinetic=False)
    eng = _engine([mon], double=True)
    eng.compute(b)
    eng._call_hooks(DynamicsStage.AFTER_STEP, b)              # first observation is the reference
    assert mon.last_drift is None
    b.energy[1] += 5e-4
    eng._call_hooks(DynamicsStage.AFTER_STEP, b)
    assert mon.last_drift.tolist() == pytest.approx([0.0, 5e-4])
    b.energy[1] += 1e-3
    with pytest.raises(RuntimeError, match="exceeds threshold"):
        eng._call_hooks(DynamicsStage.AFTER_STEP, b)
    per = EnergyDriftMonitorHook(1e-9, metric="per_atom_per_step", action="warn", include_kinetic=True)
    eng2 = _engine([per], double=True)
    eng2.compute(b)
    eng2._call_hooks(DynamicsStage.AFTER_STEP, b)
    eng2.step_count = 10
    b.velocities[0, 0] += 1.0                                 # kinetic energy of graph 0 changes
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        eng2._call_hooks(DynamicsStage.AFTER_STEP, b)
    assert any("Energy drift" in str(w.message) for w in caught)
    dke = 0.5 * float(b.atomic_masses[0]) * 1.0
    assert float(per.last_drift[0]) == pytest.approx(dke / (4 * 10), rel=1e-6) and float(per.last_drift[1]) == 0.0


def test_frozen_atoms_keep_position_and_zero_velocity_through_a_run():
    b = random_batch([6], dtype=torch.float64)
    cats = b.atom_categories.clone()
    cats[[1, 4]] = -1
    b["atom_categories"] = cats
    _ops.initialize_velocities(b.velocities, b.atomic_masses, 500.0, b.batch_idx, random_seed=1)
    p0 = b.positions.clone()
    eng = _engine([FreezeAtomsHook()], dt=1.0, double=True)
    eng.run(b, 5)
    assert torch.equal(b.positions[[1, 4]], p0[[1, 4]]) and float(b.velocities[[1, 4]].abs().sum()) == 0.0
    assert float(b.forces[[1, 4]].abs().sum()) == 0.0
    moved = (b.positions - p0).abs().sum(-1)
    assert bool((moved[[0, 2, 3, 5]] > 0).all())
    keep = FreezeAtomsHook(zero_forces=False)
    eng2 = _engine([keep], double=True)
    eng2.compute(b)
    eng2._call_hooks(DynamicsStage.AFTER_COMPUTE, b)
    assert float(b.forces[[1, 4]].abs().sum()) > 0.0          # forces stay visible (e.g. for constraint-force analysis)


def test_wrap_periodic_hook_wraps_only_periodic_directions():
    cell = torch.diag(torch.tensor([4.0, 5.0, 6.0]))
    pos = torch.tensor([[4.5, -0.5, 7.0], [1.0, 2.0, 3.0], [-8.5, 10.5, -0.25]])
    def make(pbc):
        return Batch.from_data_list([AtomicData(atomic_numbers=torch.tensor([1, 1, 1]), positions=pos.clone(), cell=cell.clone(),
                                                pbc=torch.tensor(pbc))])
    b = make([True, True, False])
    eng = _engine([WrapPeriodicHook()])
    eng._call_hooks(DynamicsStage.AFTER_POST_UPDATE, b)
    want = torch.tensor([[0.5, 4.5, 7.0], [1.0, 2.0, 3.0], [3.5, 0.5, -0.25]])
    assert torch.allclose(b.positions, want, atol=1e-6)
    open_box = make([False, False, False])
    eng._call_hooks(DynamicsStage.AFTER_POST_UPDATE, open_box)
    assert torch.equal(open_box.positions, pos)
    # displacements by whole lattice vectors: images of the same point wrap to the same place
    tri = torch.tensor([[4.0, 0.0, 0.0], [1.5, 5.0, 0.0], [-1.0, 2.0, 6.0]])
    base = torch.rand(5, 3) @ tri
    shifts = torch.randint(-3, 4, (5, 3)).float() @ tri
    bt = Batch.from_data_list([AtomicData(atomic_numbers=torch.ones(5, dtype=torch.long), positions=base + shifts, cell=tri,
                                          pbc=torch.tensor([True, True, True]))])
    eng._call_hooks(DynamicsStage.AFTER_POST_UPDATE, bt)
    assert torch.allclose(bt.positions, base, atol=1e-4)
    frac = bt.positions @ torch.linalg.inv(tri)
    assert bool(((frac > -1e-5) & (frac < 1 + 1e-5)).all())


def test_converged_snapshot_writes_only_the_converged_systems():
    b = random_batch([3, 4, 5])
    sink = HostMemory()
    hook = ConvergedSnapshotHook(sink)
    eng = _engine([hook])
    eng.compute(b)
    ctx = eng._build_context(b)
    ctx.converged_mask = torch.tensor([False, False, False])
    hook(ctx, DynamicsStage.ON_CONVERGE)
    assert len(sink) == 0
    ctx.converged_mask = torch.tensor([True, False, True])
    hook(ctx, DynamicsStage.ON_CONVERGE)
    assert len(sink) == 2
    got = sink.read()
    assert sorted(got.num_nodes_per_graph.tolist()) == [3, 5]
