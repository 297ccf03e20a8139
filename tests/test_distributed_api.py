# SPDX-License-Identifier: Apache-2.0
"""Generic domain-decomposition layer: partitioner, halo plan, sharded batch, distributed model, DomainParallel.

Multi-rank cases run as gloo processes on CPU and are compared with the single-process result."""
import os

import pytest
import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.distributed import (DistributedModel, DomainConfig, DomainParallel, HookScope, IndexPartitioner,
                                                ShardedBatch, SpatialPartitioner, factor_grid, halo_forward,
                                                halo_scatter_correct)
from nvalchemi_toolkit_b200.dynamics import NVE
from nvalchemi_toolkit_b200.hooks import NeighborListHook
from nvalchemi_toolkit_b200.models.base import BaseModelMixin
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
from tests.helpers import fcc_supercell

A = 5.26  # fcc argon-like lattice constant for the LJ cases


def _lj_batch(n_cells=4, noise=0.05, seed=0, velocities=0.0):
    d = fcc_supercell(n_cells, a=A, z=18, noise=noise, seed=seed, dtype=torch.float64)
    b = Batch.from_data_list([d])
    g = torch.Generator().manual_seed(seed + 1)
    b["velocities"] = velocities * torch.randn(b.num_nodes, 3, generator=g, dtype=torch.float64)
    return b


def _lj():
    m = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0, switch_width=1.0)
    m.model_config.active_outputs = {"energy", "forces", "stress"}
    return m


def _reference(model, batch, skin=0.0):
    from types import SimpleNamespace

    hook = NeighborListHook(model.model_config.neighbor_config, skin=skin)
    hook(SimpleNamespace(batch=batch), None)
    return model(batch)


def test_factor_grid_and_partitioner():
    assert factor_grid(8, (10.0, 10.0, 10.0)) == (2, 2, 2)
    assert factor_grid(4, (40.0, 10.0, 10.0)) == (4, 1, 1)
    cell, pbc = torch.eye(3) * 20.0, torch.tensor([True, True, True])
    part = SpatialPartitioner(cell, pbc, 4, cutoff=5.0, grid_dims=(2, 2, 1), hysteresis=0.5)
    pos = torch.tensor([[1.0, 1.0, 1.0], [11.0, 1.0, 3.0], [1.0, 11.0, 3.0], [19.0, 19.0, 0.0], [-1.0, 1.0, 1.0]])
    assert part.assign_atoms_to_ranks(pos).tolist() == [0, 2, 1, 3, 2]
    assert part.neighbor_ranks(0) == [1, 2, 3]
    # an atom just outside its owner's box stays with the owner (hysteresis), farther out it does not
    owner = torch.tensor([0, 0])
    keep = part.keeps_owner(torch.tensor([[10.3, 1.0, 1.0], [10.8, 1.0, 1.0]]), owner)
    assert keep.tolist() == [True, False]
    keep = part.keeps_owner(torch.tensor([[19.8, 1.0, 1.0]]), torch.tensor([0]))  # across the periodic boundary
    assert keep.tolist() == [True]
    ip = IndexPartitioner(10, 3)
    assert [ip.block(r) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    assert ip.owner(torch.tensor([0, 3, 4, 9])).tolist() == [0, 0, 1, 2]


def test_single_rank_periodic_images_match_pbc_model():
    batch = _lj_batch(3)
    model = _lj()
    ref = _reference(model, batch.clone())
    cfg = DomainConfig(cutoff=6.0, skin=0.0)
    sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
    assert sh.n_owned == batch.num_nodes and sh.n_ghost > 0
    out = DistributedModel(model, cfg)(sh)
    assert torch.allclose(out["forces"], ref["forces"], atol=1e-10)
    assert torch.allclose(out["energy"], ref["energy"], atol=1e-9)
    assert torch.allclose(out["stress"], ref["stress"], atol=1e-10)


def test_single_rank_weighted_energy_mace_matches_pbc_model():
    from nvalchemi_toolkit_b200.models.mace import MACEWrapper
    from nvalchemi_toolkit_b200.models.mace.model import MACE, MACEConfig

    torch.manual_seed(0)
    d = fcc_supercell(2, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)
    batch = Batch.from_data_list([d])
    model = MACEWrapper(MACE(MACEConfig(r_max=3.0, channels=8, max_ell=3, atomic_numbers=[29], radial_mlp=[16, 16],
                                        avg_num_neighbors=12.0), backend="torch")).double()
    model.model_config.active_outputs = {"energy", "forces", "stress"}
    ref = _reference(model, batch.clone())
    cfg = DomainConfig(cutoff=3.0, skin=0.0)
    sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
    out = DistributedModel(model, cfg)(sh)
    assert torch.allclose(out["energy"].reshape(-1), ref["energy"].reshape(-1), atol=1e-8)
    assert torch.allclose(out["forces"], ref["forces"], atol=1e-8)
    assert torch.allclose(out["stress"].reshape(3, 3), ref["stress"].reshape(3, 3), atol=1e-8)


def test_halo_autograd_primitives_single_rank():
    batch = _lj_batch(2)
    cfg = DomainConfig(cutoff=4.0)
    sh = ShardedBatch.from_batch(batch, cfg)
    x = torch.randn(sh.n_owned, 3, dtype=torch.float64, requires_grad=True)
    w = torch.randn(sh.n_owned + sh.n_ghost, 3, dtype=torch.float64)
    (halo_forward(x, sh.halo) * w).sum().backward()
    expect = w[: sh.n_owned].clone().index_add_(0, sh.halo.send_index, w[sh.n_owned:])
    assert torch.allclose(x.grad, expect)
    p = torch.randn(sh.n_owned + sh.n_ghost, 2, dtype=torch.float64, requires_grad=True)
    y = halo_scatter_correct(p, sh.halo)
    assert torch.allclose(y, p[: sh.n_owned].detach().clone().index_add_(0, sh.halo.send_index, p[sh.n_owned:].detach()))
    v = torch.randn_like(y)
    (y * v).sum().backward()
    assert torch.allclose(p.grad, torch.cat([v, v[sh.halo.send_index]]))


# ------------------------------------------------------------------ multi-rank (gloo)
def _md_worker(rank, world, port, q, n_steps, vel, skin, grid):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        batch = _lj_batch(4, velocities=vel)
        dyn = NVE(_lj(), dt=2.0)
        cfg = DomainConfig(cutoff=6.0, skin=skin, grid_dims=grid)
        dp = DomainParallel(dyn, cfg)
        seen = []

        class Probe:
            frequency, stage = 5, None

            def __call__(self, ctx, stage):
                seen.append((ctx.step_count, ctx.batch.num_nodes))

        from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

        dp.register_hook(Probe(), DynamicsStage.AFTER_STEP, HookScope.RANK_ZERO)
        sh = dp.run(batch, n_steps=n_steps)
        full = dp.gather()
        q.put((rank, full.positions.tolist(), full.velocities.tolist(), float(full.energy.reshape(-1)[0]), sh.num_migrated,
               dp.num_rebuilds, seen, sh.n_owned))
    finally:
        dist.destroy_process_group()


def _run_md(world, port, n_steps, vel, skin, grid):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_md_worker, args=(r, world, port, q, n_steps, vel, skin, grid)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        item = q.get(timeout=240)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    return res


def _single_md(n_steps, vel):
    batch = _lj_batch(4, velocities=vel)
    model = _lj()
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    dyn = NVE(model, dt=2.0, hooks=[NeighborListHook(model.model_config.neighbor_config, skin=0.0,
                                                     stage=DynamicsStage.BEFORE_COMPUTE)])

    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    dyn.run(batch, n_steps=n_steps)
    return batch


@pytest.mark.parametrize("world,grid", [(2, None), (4, (2, 2, 1))])
def test_domain_parallel_nve_matches_single_process(world, grid):
    n_steps, vel = 20, 0.02
    res = _run_md(world, 29610 + world, n_steps, vel, 1.0, grid)
    ref = _single_md(n_steps, vel)
    pos0 = torch.tensor(res[0][0], dtype=torch.float64)
    for r in range(1, world):  # every rank gathers the same global batch
        assert torch.equal(pos0, torch.tensor(res[r][0], dtype=torch.float64))
    assert torch.allclose(pos0, ref.positions, atol=1e-9)
    assert torch.allclose(torch.tensor(res[0][1], dtype=torch.float64), ref.velocities, atol=1e-9)
    assert abs(res[0][2] - float(ref.energy.reshape(-1)[0])) < 1e-9
    assert sum(res[r][6] for r in range(world)) == ref.num_nodes
    assert res[0][5] == [(0, 256), (5, 256), (10, 256), (15, 256)] and res[1][5] == []
    assert res[0][4] < n_steps  # the skin spared most rebuilds


def test_domain_parallel_migration_keeps_trajectory():
    n_steps, vel = 30, 0.25  # fast atoms: several cross sub-domain boundaries
    res = _run_md(2, 29640, n_steps, vel, 0.6, None)
    ref = _single_md(n_steps, vel)
    assert res[0][3] > 0  # atoms changed owner
    assert torch.allclose(torch.tensor(res[0][0], dtype=torch.float64), ref.positions, atol=1e-8)
    assert sum(res[r][6] for r in range(2)) == ref.num_nodes


def _mace_model():
    from nvalchemi_toolkit_b200.models.mace import MACEWrapper
    from nvalchemi_toolkit_b200.models.mace.model import MACE, MACEConfig

    torch.manual_seed(0)
    model = MACEWrapper(MACE(MACEConfig(r_max=3.0, channels=8, max_ell=3, atomic_numbers=[29], radial_mlp=[16, 16],
                                        avg_num_neighbors=12.0), backend="torch")).double()
    model.model_config.active_outputs = {"energy", "forces", "stress"}
    return model


def _mace_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
        model = _mace_model()
        cfg = DomainConfig(cutoff=3.0, skin=0.0)
        sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
        out = DistributedModel(model, cfg)(sh)
        from nvalchemi_toolkit_b200.distributed import ShardTensor

        forces = ShardTensor(out["forces"], sh).full_tensor()
        q.put((rank, forces.tolist(), out["energy"].reshape(-1).tolist(), out["stress"].reshape(-1).tolist(), sh.n_ghost))
    finally:
        dist.destroy_process_group()


def test_weighted_energy_reverse_halo_two_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_mace_worker, args=(r, 2, 29655, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        item = q.get(timeout=240)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
    ref = _reference(_mace_model(), batch)
    for r in range(2):
        assert torch.allclose(torch.tensor(res[r][0], dtype=torch.float64), ref["forces"], atol=1e-8)
        assert abs(res[r][1][0] - float(ref["energy"].detach().reshape(-1)[0])) < 1e-8
        assert torch.allclose(torch.tensor(res[r][2], dtype=torch.float64), ref["stress"].reshape(-1), atol=1e-8)
        assert res[r][3] > 0


def _pipe_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        pipe = _lj() + LennardJonesModelWrapper(epsilon=0.02, sigma=3.0, cutoff=3.5, switch_width=0.5)
        pipe.model_config.active_outputs = {"energy", "forces"}
        dp = DomainParallel(NVE(pipe, dt=2.0), DomainConfig(cutoff=6.0, skin=0.5))
        sh = dp.run(_lj_batch(4, velocities=0.05), n_steps=8)
        widths = sorted([sh.halo.width] + [h.width for h in sh._extra_halos.values()])
        q.put((rank, dp.gather().positions.tolist(), widths))
    finally:
        dist.destroy_process_group()


def test_domain_parallel_pipeline_model_uses_member_halos():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pipe_worker, args=(r, 2, 29671, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        item = q.get(timeout=240)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    pipe = _lj() + LennardJonesModelWrapper(epsilon=0.02, sigma=3.0, cutoff=3.5, switch_width=0.5)
    pipe.model_config.active_outputs = {"energy", "forces"}
    batch = _lj_batch(4, velocities=0.05)
    dyn = NVE(pipe, dt=2.0, hooks=pipe.make_neighbor_hooks())
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    dyn.run(batch, n_steps=8)
    assert torch.allclose(torch.tensor(res[0][0], dtype=torch.float64), batch.positions, atol=1e-9)
    assert len(res[0][1]) == 2 and res[0][1][0] < res[0][1][1]  # the short-ranged member got a shallower halo


def _val_lj():
    return _lj()


def _val_batch():
    return _lj_batch(4)


def test_trace_and_validate_passes_and_suggests_a_deeper_halo():
    from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec
    from nvalchemi_toolkit_b200.distributed.validate import trace_and_validate

    rep = trace_and_validate(_val_lj, _val_batch, 2, cutoff=6.0, port=29741)
    assert rep.ok and rep.attempts[0]["atoms_with_missing_neighbors"] == 0 and "PASS" in str(rep)
    # a spec that claims no neighbour dependence gets no ghosts: wrong forces, and the repair is a deeper halo
    bad = MLIPSpec("too_shallow", message_passes=0, consolidation=Consolidation.DIRECT_MASKED)
    rep = trace_and_validate(_val_lj, _val_batch, 2, cutoff=6.0, spec=bad, port=29751)
    assert not rep.ok and rep.suggestion == "message_passes=1 (deeper halo)"


def _gp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.distributed.strategy import get_strategy
        from nvalchemi_toolkit_b200.distributed.config import StrategyKind

        torch.set_num_threads(1)
        out = {}
        for name, model, batch in (("lj", _lj(), _lj_batch(3)), ("mace", _mace_model(), Batch.from_data_list(
                [fcc_supercell(3, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)]))):
            strat = get_strategy(DomainConfig(cutoff=6.0, strategy=StrategyKind.GRAPH_PARTITION))
            res = strat.run_forward(model, batch, model.distribution_spec())
            out[name] = {k: res[k].tolist() for k in ("energy", "forces")}
            out[name]["edges_owned"] = strat.last_edges_owned
            out[name]["n_owned"], out[name]["n_ghost"] = strat._sharded.n_owned, strat._sharded.n_ghost
        # the same partition under the dynamics wrapper
        from nvalchemi_toolkit_b200.distributed import DomainParallel
        from nvalchemi_toolkit_b200.dynamics import NVE

        dp = DomainParallel(NVE(_lj(), dt=1.0), DomainConfig(cutoff=6.0, skin=0.5, strategy=StrategyKind.GRAPH_PARTITION))
        dp.run(_lj_batch(3), n_steps=3)
        full = dp.gather()
        out["nve_positions"] = full.positions.tolist()
        out["dp_sharded"] = type(dp.sharded).__name__
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def test_graph_partition_strategy_matches_single_process():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gp_worker, args=(r, 2, 29761, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    refs = {"lj": _reference(_lj(), _lj_batch(3)),
            "mace": _reference(_mace_model(), Batch.from_data_list(
                [fcc_supercell(3, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)]))}
    for name, ref in refs.items():
        for r in range(2):
            assert torch.allclose(torch.tensor(res[r][name]["forces"], dtype=torch.float64), ref["forces"].detach(), atol=1e-8)
            assert torch.allclose(torch.tensor(res[r][name]["energy"], dtype=torch.float64), ref["energy"].detach(), atol=1e-8)
        # the work is split: each rank holds about half of the atoms and evaluates about half of the edges
        e0, e1 = res[0][name]["edges_owned"], res[1][name]["edges_owned"]
        assert e0 > 0 and e1 > 0 and 0.4 < e0 / (e0 + e1) < 0.6
        n_total = res[0][name]["n_owned"] + res[1][name]["n_owned"]
        assert abs(res[0][name]["n_owned"] - res[1][name]["n_owned"]) <= 1 and n_total == ref["forces"].shape[0]
    # NVE through DomainParallel(strategy=graph_partition) against the single-process trajectory
    from nvalchemi_toolkit_b200.dynamics import NVE, DynamicsStage

    model = _lj()
    b = _lj_batch(3)
    dyn = NVE(model, dt=1.0, hooks=model.make_neighbor_hooks())
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, b)
    dyn.compute(b)
    dyn.run(b, 3)
    for r in range(2):
        assert res[r]["dp_sharded"] == "GraphShardedBatch"
        assert torch.allclose(torch.tensor(res[r]["nve_positions"], dtype=torch.float64), b.positions, atol=1e-9)


def test_shard_routing_tables():
    from nvalchemi_toolkit_b200.distributed.context import (NOT_DISTRIBUTED, DistributedContext, ShardRouting,
                                                            activate_dd_context, current_dd_context)

    r = ShardRouting.from_assignment(torch.tensor([1, 0, 1, 2, 0]), 3)
    assert r.counts.tolist() == [2, 2, 1] and r.local_index.tolist() == [0, 0, 1, 0, 1]
    assert r.to_flat(torch.tensor([1, 4, 0, 2, 3])).tolist() == [0, 1, 2, 3, 4] and r.global_ids_of(1).tolist() == [0, 2]
    assert current_dd_context() is NOT_DISTRIBUTED
    with activate_dd_context(DistributedContext(rank=1, world_size=4, n_owned=3, n_padded=5, is_halo=True)) as c:
        assert current_dd_context().n_ghost == 2 and c.is_halo
    assert current_dd_context().world_size == 1


def _langevin_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.dynamics import NVTLangevin

        torch.set_num_threads(1)
        dp = DomainParallel(NVTLangevin(_lj(), dt=2.0, temperature=80.0, friction=0.05, random_seed=11),
                            DomainConfig(cutoff=6.0, skin=0.6))
        dp.run(_lj_batch(4, velocities=0.05), n_steps=15)
        q.put((rank, dp.gather().positions.tolist()))
    finally:
        dist.destroy_process_group()


def test_langevin_noise_follows_global_atom_ids():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics import NVTLangevin
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_langevin_worker, args=(r, 2, 29781, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    batch = _lj_batch(4, velocities=0.05)
    model = _lj()
    dyn = NVTLangevin(model, dt=2.0, temperature=80.0, friction=0.05, random_seed=11,
                      hooks=[NeighborListHook(model.model_config.neighbor_config, stage=DynamicsStage.BEFORE_COMPUTE)])
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    dyn.run(batch, n_steps=15)
    assert torch.allclose(torch.tensor(res[0], dtype=torch.float64), batch.positions, atol=1e-9)


def _npt_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.dynamics import NPT

        torch.set_num_threads(1)
        dp = DomainParallel(NPT(_lj(), dt=2.0, temperature=60.0, pressure=0.0, barostat_time=200.0, thermostat_time=50.0),
                            DomainConfig(cutoff=6.0, skin=0.6))
        dp.run(_lj_batch(4, velocities=0.05), n_steps=12)
        full = dp.gather()
        q.put((rank, full.positions.tolist(), full.cell.reshape(3, 3).tolist()))
    finally:
        dist.destroy_process_group()


def test_npt_barostat_under_domain_decomposition():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics import NPT
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_npt_worker, args=(r, 2, 29791, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r, (pos, cell)) for r, pos, cell in (q.get(timeout=240) for _ in range(2)))
    for p in procs:
        p.join(timeout=30)
    batch = _lj_batch(4, velocities=0.05)
    model = _lj()
    dyn = NPT(model, dt=2.0, temperature=60.0, pressure=0.0, barostat_time=200.0, thermostat_time=50.0,
              hooks=[NeighborListHook(model.model_config.neighbor_config, stage=DynamicsStage.BEFORE_COMPUTE)])
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    dyn.run(batch, n_steps=12)
    cell = torch.tensor(res[0][1], dtype=torch.float64)
    assert float((cell - batch.cell.reshape(3, 3)).abs().max()) < 1e-9 and float((cell - torch.eye(3) * A * 4).abs().max()) > 1e-4
    assert torch.allclose(torch.tensor(res[0][0], dtype=torch.float64), batch.positions, atol=1e-8)
    assert res[0][1] == res[1][1]


def _coll_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.distributed.collectives import (distributed_index_select, distributed_scatter_add,
                                                                    gather_to_replicate)
        from nvalchemi_toolkit_b200.distributed.context import ShardRouting

        owner = torch.tensor([0, 2, 1, 0, 2, 2, 1, 0, 1, 2])
        routing = ShardRouting.from_assignment(owner, world)
        mine = routing.global_ids_of(rank)
        table = torch.arange(10, dtype=torch.float64)[:, None] * torch.tensor([1.0, 10.0])
        local = table[mine].clone()
        ask = torch.tensor([9, 0, 4, 4, 7][rank:]) if rank else torch.tensor([3, 8, 1])
        got = distributed_index_select(local, ask, routing)
        ok_sel = torch.equal(got, table[ask])
        acc = torch.zeros(mine.numel(), 2, dtype=torch.float64)
        distributed_scatter_add(acc, torch.tensor([0, 5, 5, 8]), torch.full((4, 2), float(rank + 1), dtype=torch.float64), routing)
        full = gather_to_replicate(acc, mine)
        q.put((rank, ok_sel, full[:, 0].tolist()))
    finally:
        dist.destroy_process_group()


def test_collectives_by_global_id_and_spec_roundtrip(tmp_path):
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.distributed import SPEC_MACE_HALO, MLIPSpec
    from nvalchemi_toolkit_b200.distributed._runtime import collective_device, resolve_global_rank, resolve_world_size

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_coll_worker, args=(r, 3, 29841, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = {r: (ok, full) for r, ok, full in (q.get(timeout=120) for _ in range(3))}
    for p in procs:
        p.join(timeout=30)
    want = [0.0] * 10
    want[0], want[5], want[8] = 6.0, 12.0, 6.0  # every rank adds (rank+1) once to ids 0 and 8, twice to id 5
    for r in range(3):
        assert res[r][0] and res[r][1] == want
    SPEC_MACE_HALO.save(tmp_path / "spec.json")
    assert MLIPSpec.load(tmp_path / "spec.json") == SPEC_MACE_HALO
    assert resolve_world_size() == 1 and resolve_global_rank() == 0 and collective_device().type == "cpu"
    with pytest.warns(DeprecationWarning):
        from nvalchemi_toolkit_b200.dynamics.hooks.profiling import StageTimingHook  # noqa: F401


def _fire_worker(rank, world, port, q, kind):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.dynamics import FIRE, FIRE2, NVTNoseHoover

        torch.set_num_threads(1)
        dyn = {"fire2": lambda: FIRE2(_lj(), dt=0.05), "fire": lambda: FIRE(_lj(), dt=1.0),
               "nhc": lambda: NVTNoseHoover(_lj(), dt=2.0, temperature=60.0, thermostat_time=40.0)}[kind]()
        dp = DomainParallel(dyn, DomainConfig(cutoff=6.0, skin=0.6))
        dp.run(_lj_batch(4, noise=0.15, velocities=0.03 if kind == "nhc" else 0.0), n_steps=15)
        full = dp.gather()
        q.put((rank, full.positions.tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["fire2", "fire", "nhc"])
def test_global_reductions_of_optimisers_and_thermostats(kind):
    """FIRE's v.f / v.v / f.f sums and step limiter, and the Nose-Hoover kinetic energy and degrees of freedom, are
    global quantities: two ranks must reproduce the single-process trajectory."""
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics import FIRE, FIRE2, NVTNoseHoover
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29860 + ["fire2", "fire", "nhc"].index(kind)
    procs = [ctx.Process(target=_fire_worker, args=(r, 2, port, q, kind)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    model = _lj()
    hook = NeighborListHook(model.model_config.neighbor_config, stage=DynamicsStage.BEFORE_COMPUTE)
    dyn = {"fire2": lambda: FIRE2(model, dt=0.05, hooks=[hook]), "fire": lambda: FIRE(model, dt=1.0, hooks=[hook]),
           "nhc": lambda: NVTNoseHoover(model, dt=2.0, temperature=60.0, thermostat_time=40.0, hooks=[hook])}[kind]()
    batch = _lj_batch(4, noise=0.15, velocities=0.03 if kind == "nhc" else 0.0)
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    dyn.compute(batch)
    dyn.run(batch, n_steps=15)
    got = torch.tensor(res[0], dtype=torch.float64)
    assert float((got - batch.positions).abs().max()) < (1e-8 if kind != "fire" else 1e-6)


def _p2d_inputs():
    out = []
    for seed in (0, 1, 2):
        b = _lj_batch(4, noise=0.12, seed=seed, velocities=0.0)
        out.append(b)
    return out


def _p2d_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.distributed.pipeline2d import DomainPipeline
        from nvalchemi_toolkit_b200.dynamics import FIRE2

        torch.set_num_threads(1)
        inputs = _p2d_inputs()
        pipe = DomainPipeline([lambda: FIRE2(_lj(), dt=0.05), lambda: NVE(_lj(), dt=2.0)], n_steps=[10, 5],
                              config=DomainConfig(cutoff=6.0, skin=0.6), domain_size=2, template=inputs[0])
        res = pipe.run(inputs if rank == 0 else None)
        q.put((rank, pipe.stage, pipe.num_processed, [r.positions.tolist() for r in res]))
    finally:
        dist.destroy_process_group()


def test_pipeline_of_domain_decomposed_stages():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics import FIRE2
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_p2d_worker, args=(r, 4, 29881, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = {r: (st, n, out) for r, st, n, out in (q.get(timeout=300) for _ in range(4))}
    for p in procs:
        p.join(timeout=30)
    assert [res[r][0] for r in range(4)] == [0, 0, 1, 1] and all(res[r][1] == 3 for r in range(4))
    assert len(res[2][2]) == 3 and res[0][2] == [] and res[3][2] == []
    for k, batch in enumerate(_p2d_inputs()):  # the same two stages applied one after the other in one process
        for make, n in ((lambda m, h: FIRE2(m, dt=0.05, hooks=[h]), 10), (lambda m, h: NVE(m, dt=2.0, hooks=[h]), 5)):
            model = _lj()
            dyn = make(model, NeighborListHook(model.model_config.neighbor_config, stage=DynamicsStage.BEFORE_COMPUTE))
            dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
            dyn.compute(batch)
            dyn.run(batch, n_steps=n)
        assert torch.allclose(torch.tensor(res[2][2][k], dtype=torch.float64), batch.positions, atol=1e-8)


def test_force_strategy_and_compile_policy_round_trip(tmp_path):
    from nvalchemi_toolkit_b200.distributed import CompilePolicy, ForceStrategy
    from nvalchemi_toolkit_b200.distributed.spec import SPEC_LJ_HALO, SPEC_MACE_HALO

    assert SPEC_LJ_HALO.force_strategy is ForceStrategy.MODEL_INTERNAL
    assert SPEC_MACE_HALO.force_strategy is ForceStrategy.FRAMEWORK_FROM_NODE_ENERGY
    pol = CompilePolicy(force_strategy=ForceStrategy.FRAMEWORK_FROM_GLOBAL_ENERGY, stress_via_strain=True)
    assert pol.forces_via_autograd and not pol.consolidate_node_energy and pol.energy_output == "energy"
    assert CompilePolicy(force_strategy=ForceStrategy.FRAMEWORK_FROM_NODE_ENERGY).energy_output == "atomic_energies"
    spec = SPEC_MACE_HALO.with_(name="mace_global", compile=pol)
    assert spec.force_strategy is ForceStrategy.FRAMEWORK_FROM_GLOBAL_ENERGY
    spec.save(str(tmp_path / "spec.json"))
    back = type(spec).load(str(tmp_path / "spec.json"))
    assert back.compile == pol and back.name == "mace_global" and back.message_passes == 2


def _static_halo_checks(sh, seed):
    """Fixed-shape refresh / fold against the variable-shape primitives on the same plan (values and gradients)."""
    from nvalchemi_toolkit_b200.distributed.static_halo import (StaticHaloRouting, halo_forward_static,
                                                                halo_scatter_correct_static)

    halo, n, ng = sh.halo, sh.n_owned, sh.n_ghost
    max_send = max(max(halo.send_splits, default=0), max(halo.recv_splits, default=0)) + 3
    if dist.is_initialized():
        t = torch.tensor([max_send])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        max_send = int(t)
    n_pad = n + ng + 5
    routing = StaticHaloRouting.from_halo(halo, n, max_send, n_pad)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 3, dtype=torch.float64, generator=g)
    w = torch.randn(n + ng, 3, dtype=torch.float64, generator=g)
    xd = x.clone().requires_grad_()
    ref = halo_forward(xd, halo)
    (ref * w).sum().backward()
    pad = torch.cat([x, torch.full((ng + 5, 3), 7.0, dtype=torch.float64)]).requires_grad_()  # stale ghosts, junk in unused rows
    got = halo_forward_static(pad, routing)
    assert got.shape == (n_pad, 3) and torch.allclose(got[: n + ng], ref.detach()) and bool((got[n + ng:] == 0).all())
    (got[: n + ng] * w).sum().backward()
    assert torch.allclose(pad.grad[:n], xd.grad) and bool((pad.grad[n:] == 0).all())
    p = torch.randn(n + ng, 2, dtype=torch.float64, generator=g)
    pd = p.clone().requires_grad_()
    own = halo_scatter_correct(pd, halo)                   # owners' completed sums
    full_ref = halo_forward(own, halo)                     # ... and their ghost copies
    v = torch.randn(n + ng, 2, dtype=torch.float64, generator=g)
    (full_ref * v).sum().backward()
    ps = torch.cat([p, torch.zeros(5, 2, dtype=torch.float64)]).requires_grad_()
    full = halo_scatter_correct_static(ps, routing)
    assert torch.allclose(full[: n + ng], full_ref.detach())
    (full[: n + ng] * v).sum().backward()
    assert torch.allclose(ps.grad[: n + ng], pd.grad)
    # in-place re-pack after a rebuild keeps tensor identities (a captured graph would keep reading them)
    ids = (routing.send_index.data_ptr(), routing.recv_dest.data_ptr())
    routing.update_(halo, n)
    assert ids == (routing.send_index.data_ptr(), routing.recv_dest.data_ptr())
    small = StaticHaloRouting.allocate(routing.world, 1, n_pad, "cpu", halo.group)
    if max(halo.send_splits, default=0) > 1:
        with pytest.raises(OverflowError):
            small.update_(halo, n)
    return True


def test_static_halo_single_rank():
    sh = ShardedBatch.from_batch(_lj_batch(2), DomainConfig(cutoff=4.0))
    assert _static_halo_checks(sh, 0)


def _static_halo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        sh = ShardedBatch.from_batch(_lj_batch(3), DomainConfig(cutoff=5.0, skin=0.5))
        q.put((rank, _static_halo_checks(sh, 1), sh.n_ghost))
    except Exception as exc:  # surfaces in the parent
        q.put((rank, repr(exc), 0))
    finally:
        dist.destroy_process_group()


def test_static_halo_matches_dynamic_exchange_on_two_ranks():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_static_halo_worker, args=(r, 2, 29795, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] is True for r in res), res
    assert all(r[2] > 0 for r in res)


class _ChargeNet(torch.nn.Module, BaseModelMixin):
    """Environment-dependent partial charges (no energy of its own): the upstream member of a wired group."""

    def __init__(self, cutoff: float = 3.5) -> None:
        super().__init__()
        from nvalchemi_toolkit_b200.models.base import ModelConfig, NeighborConfig, NeighborListFormat

        self.cutoff = cutoff
        self.scale = torch.nn.Parameter(torch.tensor(0.4, dtype=torch.float64))
        self.model_config = ModelConfig(outputs=frozenset({"energy", "charges"}), active_outputs={"energy", "charges"},
                                        neighbor_config=NeighborConfig(cutoff=cutoff, format=NeighborListFormat.MATRIX))

    def forward(self, data, **kw):
        pos = data.positions
        nm, num = data.neighbor_matrix.long(), data.num_neighbors.long()
        n = pos.shape[0]
        valid = torch.arange(nm.shape[1], device=nm.device)[None, :] < num[:, None]
        j = torch.where(valid, nm, torch.zeros_like(nm))
        cell = data.cell.reshape(-1, 3, 3)[data.batch_idx.long()].to(pos.dtype)
        sh = torch.einsum("nki,nij->nkj", data.neighbor_matrix_shifts.to(pos.dtype), cell)
        r = (pos[j] + sh - pos[:, None, :]).norm(dim=-1)
        w = torch.where(valid & (r < self.cutoff), torch.exp(-r) * (1.0 - r / self.cutoff) ** 2, torch.zeros_like(r)).sum(-1)
        sign = torch.where(data.atomic_numbers == 11, 1.0, -1.0).to(pos.dtype)
        nb = data.cell.reshape(-1, 3, 3).shape[0]
        return {"energy": pos.new_zeros(nb, 1) + 0.0 * w.sum(), "charges": sign * torch.tanh(self.scale * w)}

    def distribution_spec(self, strategy=None):
        from nvalchemi_toolkit_b200.distributed import Consolidation, MLIPSpec

        return MLIPSpec("charge_net", message_passes=1, consolidation=Consolidation.WEIGHTED_ENERGY)


def _wired_pipeline():
    from nvalchemi_toolkit_b200.models.ewald import EwaldModelWrapper
    from nvalchemi_toolkit_b200.models.pipeline import PipelineGroup, PipelineModelWrapper, PipelineStep

    torch.manual_seed(0)
    coulomb = EwaldModelWrapper(cutoff=5.0, accuracy=1e-6)
    lj = LennardJonesModelWrapper(epsilon=0.01, sigma=2.6, cutoff=4.5, switch_width=0.5)
    pipe = PipelineModelWrapper([PipelineGroup([PipelineStep(_ChargeNet(), wire={"charges": "node_charges"}), coulomb],
                                               use_autograd=True), PipelineGroup([lj])])
    pipe.model_config.active_outputs = {"energy", "forces"}
    return pipe


def _nacl_batch():
    from nvalchemi_toolkit_b200.benchmark import build

    return build("nacl", 2, dtype=torch.float64, noise=0.05)


def _wired_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        from nvalchemi_toolkit_b200.distributed import DistributedPipelineModel, ShardTensor

        pipe = _wired_pipeline()
        cfg = DomainConfig(cutoff=5.0, skin=0.0)
        dm = DistributedPipelineModel(pipe, cfg)
        cfg = cfg.model_copy(update={"ghost_width": dm.required_ghost_width})
        sh = ShardedBatch.from_batch(_nacl_batch(), cfg)
        out = dm(sh)
        forces = ShardTensor(out["forces"], sh).full_tensor()
        q.put((rank, forces.tolist(), float(out["energy"].reshape(-1)[0]), dm.required_ghost_width, sh.n_owned))
    except Exception as exc:
        import traceback

        q.put((rank, "".join(traceback.format_exception(exc))[-1500:], 0.0, 0.0, 0))
    finally:
        dist.destroy_process_group()


def test_wired_autograd_group_is_decomposed_as_one_model():
    """Predicted charges wired into Ewald inside an autograd group, plus a direct pair-potential group, over two ranks:
    energy and forces (including the response of the charges to the positions) match the single-process pipeline; the group's
    ghost layer is as deep as both members' ranges chained."""
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_wired_worker, args=(r, 2, 29796, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        item = q.get(timeout=300)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    assert not isinstance(res[0][0], str), res[0][0]
    pipe = _wired_pipeline()
    batch = _nacl_batch()
    dyn = NVE(pipe, dt=1.0, hooks=pipe.make_neighbor_hooks())
    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
    ref = dyn.compute(batch)
    for r in range(2):
        assert abs(res[r][1] - float(ref["energy"].reshape(-1)[0])) < 1e-8
        assert torch.allclose(torch.tensor(res[r][0], dtype=torch.float64), ref["forces"], atol=1e-8)
        assert abs(res[r][2] - 8.5) < 1e-9 and 0 < res[r][3] < batch.num_nodes


def test_static_halo_capacities_grow_only_and_repack_in_place():
    from nvalchemi_toolkit_b200.distributed.static_halo import StaticHalo

    sh = ShardedBatch.from_batch(_lj_batch(2), DomainConfig(cutoff=4.0))
    st = StaticHalo(sh.halo)
    r1 = st.sync(sh.n_owned)
    assert st.generation == 1 and r1.max_send >= max(sh.halo.send_splits) and r1.n_padded >= sh.n_owned + sh.n_ghost
    assert r1.max_send % 16 == 0 and r1.n_padded % 16 == 0
    x = torch.randn(sh.n_owned, 3, dtype=torch.float64)
    full = st.refresh(x)
    assert torch.allclose(full[: sh.n_owned + sh.n_ghost], halo_forward(x, sh.halo))
    ptr = r1.send_index.data_ptr()
    sh.halo.build(sh.owned.positions.detach(), sh.global_ids)     # same geometry, new plan generation
    r2 = st.sync(sh.n_owned)
    assert r2 is r1 and st.generation == 1 and r2.send_index.data_ptr() == ptr
    if max(sh.halo.send_splits) > 16:                             # pretend the first plan was tiny: the next sync must grow
        st.caps["max_send"], st.routing.max_send = 16, 16
        sh.halo.num_builds += 1
        r3 = st.sync(sh.n_owned)
        assert st.generation == 2 and r3.max_send > 16 and r3 is not r1


@pytest.mark.gpu
def test_static_halo_replays_in_a_cuda_graph_across_rebuilds():
    """The point of the fixed shapes: a ghost refresh captured ONCE in a CUDA graph keeps working after the exchange was
    rebuilt for moved atoms, because the routing tensors it reads are re-packed in place."""
    from nvalchemi_toolkit_b200.distributed.static_halo import StaticHalo

    batch = _lj_batch(3).to("cuda")
    sh = ShardedBatch.from_batch(batch, DomainConfig(cutoff=5.0, skin=0.5))
    st = StaticHalo(sh.halo)
    routing = st.sync(sh.n_owned)
    x = torch.randn(sh.n_owned, 4, device="cuda", dtype=torch.float64)
    static_in = st.pad(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up outside the capture
            halo_forward_static_out = st.refresh(x)
    torch.cuda.current_stream().wait_stream(side)
    from nvalchemi_toolkit_b200.distributed.static_halo import halo_forward_static

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        static_out = halo_forward_static(static_in, routing)
    graph.replay()
    torch.cuda.synchronize()
    n, ng = sh.n_owned, sh.n_ghost
    assert torch.allclose(static_out[: n + ng], halo_forward(x, sh.halo))
    # move atoms across the periodic boundary, rebuild the plan, re-pack in place, replay the SAME graph
    sh.owned.positions.add_(1.7)
    sh.halo.build(sh.owned.positions.detach(), sh.global_ids)
    assert st.sync(sh.n_owned) is routing
    x2 = torch.randn_like(x)
    static_in.zero_()
    static_in[:n].copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    ng2 = sh.halo.n_ghost
    assert torch.allclose(static_out[: n + ng2], halo_forward(x2, sh.halo)) and bool((static_out[n + ng2:] == 0).all())


def _health_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import warnings

        from nvalchemi_toolkit_b200.distributed.distributed_model import partition_health_verdict

        torch.set_num_threads(1)
        res = {}
        # every rank reaches the same verdict although only rank 1 is empty / only rank 0 is trivial
        res["verdict_empty"] = partition_health_verdict(0 if rank == 1 else 10, 12, None, "cpu")
        res["verdict_trivial"] = partition_health_verdict(10, 20 if rank == 0 else 12, None, "cpu")
        res["verdict_fine"] = partition_health_verdict(10, 14, None, "cpu")
        model = _lj()
        # 3 x 5.26 A box on two ranks with a 6 A ghost layer: each rank's halo holds every other atom
        small = _lj_batch(3)
        cfg = DomainConfig(cutoff=6.0, skin=0.0)
        sh = ShardedBatch.from_batch(small, cfg, model.distribution_spec())
        dm = DistributedModel(model, cfg)
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            dm(sh)
            dm(sh)  # checked once
        res["warned"] = sum("trivial domain decomposition" in str(w.message) for w in caught)
        res["message"] = dm.partition_health
        strict = DomainConfig(cutoff=6.0, skin=0.0, strict_partition_health=True)
        try:
            DistributedModel(model, strict)(ShardedBatch.from_batch(small, strict, model.distribution_spec()))
            res["strict"] = "ran"
        except RuntimeError as exc:
            res["strict"] = str(exc)
        # all atoms in one half of the box: the other rank would own nothing, and BOTH ranks raise
        lopsided = _lj_batch(3)
        lopsided["positions"] = lopsided.positions * torch.tensor([0.3, 1.0, 1.0], dtype=torch.float64) + torch.tensor(
            [1.0, 0.0, 0.0], dtype=torch.float64)  # x within [1, 6] A of a 15.8 A box, clear of the periodic seam
        try:
            ShardedBatch.from_batch(lopsided, DomainConfig(cutoff=6.0, skin=0.0, grid_dims=(2, 1, 1)), model.distribution_spec())
            res["empty"] = "built"
        except RuntimeError as exc:
            res["empty"] = str(exc)
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_partition_health_verdict_is_collective_and_acted_on_identically():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.distributed.distributed_model import resolve_partition_health

    # the pure part: what each verdict leads to
    assert resolve_partition_health(False, False, 100, world_size=4, strict=True, rank=0) is None
    with pytest.raises(RuntimeError, match="owns no atoms"):
        resolve_partition_health(True, False, 100, world_size=4, strict=False, rank=2)
    with pytest.raises(RuntimeError, match="strict_partition_health"):
        resolve_partition_health(False, True, 100, world_size=4, strict=True, rank=1)
    assert resolve_partition_health(False, True, 100, world_size=1, strict=True, rank=0) is None  # one rank: nothing to gain anyway
    with pytest.warns(RuntimeWarning, match="trivial domain decomposition"):
        msg = resolve_partition_health(False, True, 100, world_size=2, strict=False, rank=0)
    assert "100 atoms" in msg

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_health_worker, args=(r, 2, 29697, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    for r in range(2):
        assert res[r]["verdict_empty"] == (True, True, 10)   # 10 atoms in total, and rank 0's 12 padded rows cover them
        assert res[r]["verdict_trivial"] == (False, True, 20) and res[r]["verdict_fine"] == (False, False, 20)
        assert "trivial domain decomposition" in res[r]["message"]
        assert "strict_partition_health" in res[r]["strict"]
        assert "own no atoms" in res[r]["empty"] and "[1]" in res[r]["empty"]
    assert res[0]["warned"] == 1 and res[1]["warned"] == 0  # rank 0 speaks, once


def _coo_pair_model():
    """A pair potential that reads an EDGE LIST (``NeighborListFormat.COO``) and knows nothing about decomposition."""
    from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec
    from nvalchemi_toolkit_b200.models.base import ModelConfig, NeighborConfig, NeighborListFormat

    class CooPair(torch.nn.Module, BaseModelMixin):
        def __init__(self):
            super().__init__()
            self.model_config = ModelConfig(outputs=frozenset({"energy", "forces"}),
                                            neighbor_config=NeighborConfig(cutoff=4.0, format=NeighborListFormat.COO))

        def forward(self, data, **kw):
            nl = data.neighbor_list.long()
            i, j = nl[:, 0], nl[:, 1]
            r = data.positions[j] - data.positions[i]
            shifts = getattr(data, "shifts", None)
            if shifts is not None:
                r = r + shifts.to(r.dtype)
            d = r.norm(dim=-1)
            n = data.positions.shape[0]
            e_atom = torch.zeros(n, dtype=r.dtype).index_add_(0, i, 0.25 * (d - 4.0) ** 2)   # half of each pair's energy
            forces = torch.zeros(n, 3, dtype=r.dtype).index_add_(0, i, ((d - 4.0) / d)[:, None] * r)
            energy = torch.zeros(data.num_graphs, dtype=r.dtype).index_add_(0, data.batch_idx.long(), e_atom)
            return {"energy": energy.reshape(-1, 1), "forces": forces}

        def distribution_spec(self, strategy=None):
            return MLIPSpec("coo_pair", message_passes=1, consolidation=Consolidation.DIRECT_MASKED)

    return CooPair()


def test_edge_list_model_keeps_only_edges_of_owned_receivers():
    """One rank, periodic images as ghosts: every edge between two local atoms exists in the padded edge list, and only
    those whose receiver is owned may count; energy and forces equal the periodic single-process evaluation."""
    model = _coo_pair_model()
    batch = Batch.from_data_list([fcc_supercell(3, a=3.9, z=29, noise=0.1, seed=5, dtype=torch.float64)])
    ref = _reference(model, batch.clone())
    cfg = DomainConfig(cutoff=4.0, skin=0.0)
    sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
    dm = DistributedModel(model, cfg)
    out = dm(sh)
    assert sh.n_ghost > 0
    assert torch.allclose(out["forces"], ref["forces"], atol=1e-10) and torch.allclose(out["energy"], ref["energy"], atol=1e-9)
    # without the filter the ghost receivers' edges would have been counted as well
    padded = sh.padded_batch(sh.halo)
    dm.neighbor_hook._bufs = None
    from types import SimpleNamespace

    dm.neighbor_hook(SimpleNamespace(batch=padded), None)
    every = int(padded.neighbor_list.shape[0])
    kept = int((padded.neighbor_list[:, 0] < sh.n_owned).sum())
    assert kept == int(ref_edges(batch, model)) and every > kept


def ref_edges(batch, model):
    from types import SimpleNamespace

    b = batch.clone()
    NeighborListHook(model.model_config.neighbor_config)(SimpleNamespace(batch=b), None)
    return b.neighbor_list.shape[0]


def _helpers_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.distributed import helpers

        torch.set_num_threads(1)
        model = _lj()
        batch = _lj_batch(4)
        cfg = DomainConfig(cutoff=6.0, skin=0.0)
        sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
        n, ng = sh.n_owned, sh.n_ghost
        gid = sh.global_ids
        res = {"n": n, "ng": ng}
        # a per-atom quantity known globally: f(global id)
        feat = torch.stack([gid.double(), (gid * gid).double()], dim=1)
        padded = helpers.refresh_ghosts(feat, sh)
        ghost_gid = sh.halo.forward(gid.double().reshape(-1, 1)).reshape(-1).long()
        res["refresh_ok"] = bool(torch.equal(padded[:n], feat) and torch.equal(padded[n:, 1], (ghost_gid * ghost_gid).double()))
        # ghost rows each contribute 1: an owner receives as many as it has copies elsewhere; the total is conserved
        back = helpers.scatter_to_owners(torch.ones(ng, 1, dtype=torch.float64), torch.zeros(n, 1, dtype=torch.float64), sh)
        total = back.sum().reshape(1)
        dist.all_reduce(total)
        ghosts = torch.tensor([float(ng)])
        dist.all_reduce(ghosts)
        res["scatter_total"], res["ghost_total"] = float(total), float(ghosts)
        # weighted per-system sums over owned + ghost rows equal the global sum once reduced
        w = sh.owned_mask().double()
        bidx = torch.zeros(n + ng, dtype=torch.long)
        s = helpers.system_sum(padded[:, 0], bidx, 1, weights=w, distributed=True)
        res["system_sum"] = float(s)
        # uniform charge shift to a target total, with global sums and counts
        q_local = torch.sin(torch.cat([gid, ghost_gid]).double())
        fixed = helpers.total_charge_correction(q_local, torch.tensor([2.5], dtype=torch.float64), bidx, weights=w, distributed=True)
        tot = (fixed * w).sum().reshape(1)
        dist.all_reduce(tot)
        res["charge_total"] = float(tot)
        res["charge_shift_uniform"] = float((fixed - q_local).std())
        rows = helpers.gather_replicated(torch.full((rank + 1, 2), float(rank)))
        res["gathered"] = rows[:, 0].tolist()
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_model_author_helpers_single_process_and_two_ranks():
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200.distributed import helpers

    # no process group: identities and plain local reductions
    x = torch.arange(6.0).reshape(3, 2)
    assert helpers.refresh_ghosts(x) is x and helpers.scatter_to_owners(torch.ones(2, 2), x) is x and helpers.to_local(x) is x
    s = helpers.system_sum(torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([0, 0, 1, 1]), 2, weights=torch.tensor([1, 0, 1, 1]))
    assert s.tolist() == [1.0, 7.0]
    fixed = helpers.total_charge_correction(torch.tensor([0.1, 0.2, 0.3, -0.2]), torch.tensor([0.0, 1.0]), torch.tensor([0, 0, 1, 1]))
    assert torch.allclose(fixed, torch.tensor([-0.05, 0.05, 0.75, 0.25]))

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_helpers_worker, args=(r, 2, 29699, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    n_total = res[0]["n"] + res[1]["n"]
    assert n_total == 256
    for r in range(2):
        assert res[r]["ng"] > 0 and res[r]["refresh_ok"]
        assert res[r]["scatter_total"] == res[r]["ghost_total"] > 0
        assert res[r]["system_sum"] == pytest.approx(n_total * (n_total - 1) / 2)
        assert res[r]["charge_total"] == pytest.approx(2.5, abs=1e-9) and res[r]["charge_shift_uniform"] < 1e-12
        assert res[r]["gathered"] == [0.0, 1.0, 1.0]
