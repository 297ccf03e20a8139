# SPDX-License-Identifier: Apache-2.0
"""``DomainParallel`` over the peer-memory engine (native MACE, ghost rows through NVLink kernels) against the
single-GPU run of the same system: slabs and 3-D rank grids, Langevin trajectory, FIRE relaxation, stress."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank: int, world: int, port: int, q, grid, channels: int) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from nvalchemi_toolkit_b200 import Batch
        from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel
        from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, DynamicsStage, NVTLangevin, _ops
        from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper
        from nvalchemi_toolkit_b200.ops import gemm
        from tests.helpers import fcc_supercell

        gemm.set_precision("fp32" if channels != 128 else "tf32")  # 128 channels: the fused tensor-core convolution
        torch.manual_seed(0)
        model = MACE(MACEConfig(atomic_numbers=[29], channels=channels, avg_num_neighbors=42.0)).to(dev)
        cells = 8

        def system():
            d = fcc_supercell(cells, noise=0.08, seed=3)
            b = Batch.from_data_list([d], device=dev)
            vel = torch.zeros(b.num_nodes, 3, device=dev)
            _ops.initialize_velocities(vel, b.atomic_masses, 300.0, b.batch_idx, random_seed=1, remove_com=False, rescale=False)
            b["velocities"] = vel
            return b

        def wrapper(outputs=("energy", "forces")):
            w = MACEWrapper(model)
            w.eval()
            w.model_config.active_outputs = set(outputs)
            return w

        res = {}
        # ---- Langevin trajectory through the public API on both sides
        cfg = DomainConfig(cutoff=5.0, skin=1.0, neighbor_skin=0.0, grid_dims=grid, peer_memory=True)
        with DomainParallel(NVTLangevin(wrapper(), dt=1.0, temperature=300.0, friction=0.01, random_seed=7), cfg,
                            max_neighbors=64) as dp:
            sh = dp.partition(system())
            dp.compute()
            e_dd = float(sh.owned.energy)
            g0 = dp.gather()
            w = wrapper()
            ref = system()
            dyn = NVTLangevin(w, dt=1.0, temperature=300.0, friction=0.01, random_seed=7, hooks=w.make_neighbor_hooks(64))
            dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, ref)
            dyn.compute(ref)
            res.update(e_err=abs(e_dd - float(ref.energy)), e=float(ref.energy),
                       f_err=float((g0.forces - ref.forces).abs().max()), f=float(ref.forces.abs().max()))
            dp.run(n_steps=3)
            dyn.run(ref, 3)
            g1 = dp.gather()
            L = float(ref.cell[0, 0, 0])
            dx = g1.positions - ref.positions
            dx = dx - L * torch.round(dx / L)
            res.update(x_err=float(dx.abs().max()), v_err=float((g1.velocities - ref.velocities).abs().max()),
                       status=dp.model.engine.status(), ghosts=sh.n_ghost, owned=sh.n_owned,
                       engine=type(dp.model.engine).__name__)
        # ---- stress (virial summed over ranks) and a short FIRE relaxation with a global convergence test
        cfg = DomainConfig(cutoff=5.0, skin=1.0, neighbor_skin=0.0, grid_dims=grid)
        with DomainParallel(FIRE(wrapper(("energy", "forces", "stress")), dt=1.0,
                                 convergence_hook=ConvergenceHook.from_fmax(1e-9)), cfg, max_neighbors=64) as dp:
            sh = dp.partition(system())
            dp.compute()
            w = wrapper(("energy", "forces", "stress"))
            ref = system()
            fire = FIRE(w, dt=1.0, hooks=w.make_neighbor_hooks(64))
            fire._call_hooks(DynamicsStage.BEFORE_COMPUTE, ref)
            fire.compute(ref)
            res["s_err"] = float((sh.owned.stress.reshape(3, 3) - ref.stress.reshape(3, 3)).abs().max())
            res["s"] = float(ref.stress.abs().max())
            dp.run(n_steps=5)
            fire.run(ref, 5)
            g = dp.gather()
            dx = g.positions - ref.positions
            dx = dx - L * torch.round(dx / L)
            res.update(fire_x_err=float(dx.abs().max()), fire_e_err=abs(float(sh.owned.energy) - float(ref.energy)),
                       converged=bool(dp.converged))
        res["gemm"] = gemm.check_errors(ref.positions)
        q.put((rank, res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, {"error": f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"}))


@pytest.mark.parametrize("world,grid,channels", [(2, (2, 1, 1), 32), (2, (1, 1, 2), 128), (4, (2, 2, 1), 128),
                                                 (8, (2, 2, 2), 128)])
def test_domain_parallel_peer_engine_matches_single_gpu(world, grid, channels):
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world * 7 + channels % 97
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, grid, channels)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=900) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    tol = 1.0 if channels != 128 else 30.0  # tf32 channel mixes against the same kernels on one GPU (summation order)
    for r, res in results.items():
        assert "error" not in res, res["error"]
        assert res["engine"] == "PeerHaloEngine" and res["status"] == 0 and res["gemm"] == 0
        assert res["owned"] > 0 and res["ghosts"] > 0
        assert res["e_err"] < 1e-3 * tol * max(1.0, abs(res["e"]))
        assert res["f_err"] < 2e-4 * tol * max(1.0, res["f"])
        assert res["x_err"] < 1e-4 * tol and res["v_err"] < 1e-4 * tol
        assert res["s_err"] < 2e-4 * tol * max(1e-3, res["s"])
        assert res["fire_x_err"] < 1e-4 * tol and res["fire_e_err"] < 1e-3 * tol * max(1.0, abs(res["e"]))
        assert not res["converged"]
    assert sum(res["owned"] for res in results.values()) == 4 * 8 ** 3
