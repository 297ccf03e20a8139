# SPDX-License-Identifier: Apache-2.0
"""Generic domain-decomposition layer over NCCL on 2 GPUs: Lennard-Jones NVE and a PME + LJ composite against the
single-GPU run of the same system."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _lj():
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

    m = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0, switch_width=1.0)
    m.model_config.active_outputs = {"energy", "forces"}
    return m


def _worker(rank: int, world: int, port: int, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from nvalchemi_toolkit_b200.benchmark import build
        from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, DomainParallel, ShardedBatch, ShardTensor
        from nvalchemi_toolkit_b200.dynamics import NVE, DynamicsStage, _ops
        from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper

        res = {}
        # ---- NVE trajectory, float64
        def system():
            b = build("fcc_cu", 6, device=dev, a=5.26, z=18, dtype=torch.float64)
            _ops.initialize_velocities(b.velocities, b.atomic_masses, 80.0, b.batch_idx, random_seed=3)
            return b

        dp = DomainParallel(NVE(_lj(), dt=2.0), DomainConfig(cutoff=6.0, skin=0.8))
        sh = dp.run(system(), n_steps=25)
        full = dp.gather()
        ref = system()
        model = _lj()
        dyn = NVE(model, dt=2.0, hooks=model.make_neighbor_hooks())
        dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, ref)
        dyn.compute(ref)
        dyn.run(ref, n_steps=25)
        res["x_err"] = float((full.positions - ref.positions).abs().max())
        res["owned"], res["ghosts"], res["rebuilds"] = sh.n_owned, sh.n_ghost, dp.num_rebuilds
        # ---- composite model with a global reciprocal sum (mesh all-reduce across ranks)
        def salt():
            return build("nacl", 4, device=dev, noise=0.05, dtype=torch.float64)

        pme = PMEModelWrapper(cutoff=6.0, accuracy=1e-7)
        pme.model_config.active_outputs = {"energy", "forces"}
        cfg = DomainConfig(cutoff=6.0, skin=0.0)
        shs = ShardedBatch.from_batch(salt(), cfg, pme.distribution_spec())
        out = DistributedModel(pme, cfg)(shs)
        forces = ShardTensor(out["forces"], shs).full_tensor()
        single = salt()
        pme2 = PMEModelWrapper(cutoff=6.0, accuracy=1e-7)
        pme2.model_config.active_outputs = {"energy", "forces"}
        from types import SimpleNamespace

        for h in pme2.make_neighbor_hooks():
            h(SimpleNamespace(batch=single), None)
        o2 = pme2(single)
        res["pme_f_err"] = float((forces - o2["forces"]).abs().max())
        res["pme_e_err"] = abs(float(out["energy"]) - float(o2["energy"]))
        from nvalchemi_toolkit_b200.parallel.symmetric import peer_reducer

        red = peer_reducer(None, dev)  # the mesh and net-charge sums of the evaluation above went through peer memory
        res["peer_reductions"], res["library_reductions"], res["peer_status"] = red.calls, red.fallbacks, red.ctx.status()
        q.put((rank, res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, {"error": f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"}))


def test_generic_domain_layer_over_nccl():
    import torch.multiprocessing as mp

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29547, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    for r, res in results.items():
        assert "error" not in res, res["error"]
        assert res["owned"] > 0 and res["ghosts"] > 0
        assert res["x_err"] < 1e-8
        assert res["pme_f_err"] < 1e-8 and res["pme_e_err"] < 1e-7
        assert res["peer_reductions"] >= 2 and res["library_reductions"] == 0 and res["peer_status"] == 0
    assert results[0]["owned"] + results[1]["owned"] == 864
