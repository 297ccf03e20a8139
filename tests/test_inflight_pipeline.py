# SPDX-License-Identifier: Apache-2.0
"""Sampler, sinks, hooks, inflight batching and the two-stage distributed pipeline (gloo ranks on CPU)."""
import os

import pytest
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.dynamics import FIRE, NVE, ConvergenceHook, DemoDynamics
from nvalchemi_toolkit_b200.dynamics.hooks import (EnergyDriftMonitorHook, FreezeAtomsHook, LoggingHook, MaxForceClampHook,
                                                   NaNDetectorHook, SnapshotHook)
from nvalchemi_toolkit_b200.dynamics.sampler import SizeAwareSampler
from nvalchemi_toolkit_b200.dynamics.sinks import GPUBuffer, HostMemory
from nvalchemi_toolkit_b200.hooks.stage_timing import StageTimingHook
from nvalchemi_toolkit_b200.models import DemoModelWrapper
from tests.helpers import random_batch, random_molecule


class ListDataset:
    def __init__(self, sizes, seed=0):
        self.items = [random_molecule(n, seed + i) for i, n in enumerate(sizes)]

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        return self.items[i].clone(), {}

    def get_metadata(self, i):
        return self.items[i].num_nodes, 0


def test_sampler_budgets_and_ids():
    ds = ListDataset([4, 9, 6, 12, 3, 7])
    s = SizeAwareSampler(ds, max_atoms=20, max_batch_size=3)
    b = s.build_initial_batch()
    assert b.num_graphs <= 3 and b.num_nodes <= 20 and b.status.shape == (b.num_graphs, 1)
    assert sorted(b.system_id.reshape(-1).tolist()) == list(range(b.num_graphs))
    more = s.request_replacements_budget(atom_budget=13, max_count=2)
    assert sum(m.num_nodes for m in more) <= 13 and len(more) <= 2
    one = s.request_replacement(5, 0)
    assert one is None or one.num_nodes <= 5
    while not s.exhausted:
        got = s.request_replacements_budget(atom_budget=100)
        assert got
    with pytest.raises(RuntimeError):
        SizeAwareSampler(ListDataset([30]), max_atoms=20)
    with pytest.raises(ValueError):
        SizeAwareSampler(ds)


def test_sinks_roundtrip():
    b = random_batch([3, 4, 5])
    for sink in (HostMemory(capacity=10), GPUBuffer(capacity=4, max_atoms=8, device="cpu")):
        sink.write(b, mask=torch.tensor([True, False, True]))
        assert len(sink) == 2 and not sink.is_full
        got = sink.read()
        assert got.num_graphs == 2 and got.num_nodes == 8
        assert torch.allclose(got.positions[:3], b.positions[:3])
        part = sink.drain(max_systems=1)
        assert part.num_graphs == 1 and len(sink) == 1
        sink.zero()
        assert len(sink) == 0


def test_stock_hooks(tmp_path):
    b = random_batch([5, 6])
    model = DemoModelWrapper()
    sink = HostMemory()
    log = LoggingHook(backend="memory", frequency=2)
    timing = StageTimingHook("all", enable_nvtx=False, timer_backend="perf_counter", log_path=tmp_path / "t.csv")
    cats = b.atom_categories.clone()
    cats[0] = -1
    b["atom_categories"] = cats
    p0 = b.positions[0].clone()
    dyn = NVE(model, dt=0.5, hooks=[NaNDetectorHook(), MaxForceClampHook(10.0), EnergyDriftMonitorHook(1.0),
                                    FreezeAtomsHook(), SnapshotHook(sink, frequency=2), log, timing])
    dyn.compute(b)
    from nvalchemi_toolkit_b200.dynamics import _ops

    _ops.initialize_velocities(b.velocities, b.atomic_masses, 300.0, b.batch_idx)
    dyn.run(b, 4)
    assert torch.equal(b.positions[0], p0)  # frozen atom
    assert len(sink) == 4  # 2 snapshots x 2 graphs
    assert [s for s, _ in log.records] == [0, 2] and "temperature" in log.records[0][1][0]
    assert len(timing.rows) == 4 and (tmp_path / "t.csv").exists() and "total_ms" in timing.summary()
    b.forces[0, 0] = float("nan")
    with pytest.raises(RuntimeError):
        NaNDetectorHook()(dyn._build_context(b), dyn.hooks[0].stage)


def test_inflight_batching_processes_every_system():
    ds = ListDataset([4, 9, 6, 12, 3, 7, 5, 8])
    sampler = SizeAwareSampler(ds, max_atoms=24, max_batch_size=3)
    sink = HostMemory()
    model = DemoModelWrapper()
    relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(1e9))
    md = NVE(model, dt=0.5, n_steps=2)
    fused = relax + md
    fused.sampler, fused.sinks = sampler, [sink]
    out = fused.run()
    assert out is None and sampler.exhausted
    done = sink.read()
    assert done.num_graphs == 8 and sorted(done.system_id.reshape(-1).tolist()) == list(range(8))
    assert sorted(done.num_nodes_list) == sorted([4, 9, 6, 12, 3, 7, 5, 8])


def _pipeline_worker(rank, world, port, q, comm_mode="async_recv"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = DemoModelWrapper()
        ds = ListDataset([4, 9, 6, 12, 3, 7])
        sampler = SizeAwareSampler(ds, max_atoms=24, max_batch_size=3)
        sink = HostMemory()
        relax = FIRE(model, dt=0.1, convergence_hook=ConvergenceHook.from_fmax(1e9), sampler=sampler, device_type="cpu",
                     max_batch_size=3, comm_mode=comm_mode)
        md = DemoDynamics(model, n_steps=3, dt=0.05, sinks=[sink], device_type="cpu", max_batch_size=8, comm_mode=comm_mode)
        pipe = relax | md
        pipe.setup()
        pipe.run(max_iterations=200)
        done = sink.read()
        q.put((rank, pipe.iterations, 0 if done is None else done.num_graphs,
               [] if done is None else sorted(done.system_id.reshape(-1).tolist())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("comm_mode", ["sync", "async_recv", "fully_async"])
def test_two_stage_pipeline_gloo(comm_mode):
    """Every communication mode (blocking hand-off, overlapped receive, overlapped receive and send) delivers every system."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29577 + ["sync", "async_recv", "fully_async"].index(comm_mode)
    procs = [ctx.Process(target=_pipeline_worker, args=(r, 2, port, q, comm_mode)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert res[0][1] == res[1][1] < 200  # both ranks ran the same number of iterations and terminated
    assert res[0][2] == 0 and res[1][2] == 6 and res[1][3] == list(range(6))
