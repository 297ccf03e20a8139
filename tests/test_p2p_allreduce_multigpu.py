# SPDX-License-Identifier: Apache-2.0
"""Peer-memory all-reduce (NVSwitch multimem path when a multicast mapping exists, peer loads otherwise) against NCCL."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank: int, world: int, port: int, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

        n = 1 << 20
        ctx = P2PContext(4 * n + 4096, dev)
        buf, _ = ctx.arena.alloc((n,), torch.float32)
        res = {"multicast": ctx.arena.multicast_ptr != 0}
        for name, mm in (("p2p", False), ("multimem", True)):
            if mm and not res["multicast"]:
                continue
            g = torch.Generator(device=dev).manual_seed(100 + rank)
            x = torch.randn(n, generator=g, device=dev)
            buf.copy_(x)
            want = x.clone()
            dist.all_reduce(want)
            got = ctx.allreduce_(buf, scale=0.5, use_multimem=mm)
            torch.cuda.synchronize()
            res[name] = float((got - 0.5 * want).abs().max())
            # timing: bytes that cross the links per rank, algorithm bandwidth
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                ctx.allreduce_(buf, use_multimem=mm)
            torch.cuda.synchronize()
            t0.record()
            for _ in range(10):
                ctx.allreduce_(buf, use_multimem=mm)
            t1.record()
            torch.cuda.synchronize()
            res[name + "_us"] = t0.elapsed_time(t1) * 100.0
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        y = torch.randn(n, device=dev)
        for _ in range(3):
            dist.all_reduce(y)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(10):
            dist.all_reduce(y)
        t1.record()
        torch.cuda.synchronize()
        res["nccl_us"] = t0.elapsed_time(t1) * 100.0
        res["status"] = ctx.status()
        q.put((rank, res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, {"error": f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"}))


def test_peer_allreduce_matches_nccl():
    import torch.multiprocessing as mp

    world = min(torch.cuda.device_count(), 8)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29561, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    for r, res in results.items():
        assert "error" not in res, res["error"]
        assert res["status"] == 0
        assert res["p2p"] < 1e-4
        if res["multicast"]:
            assert res["multimem"] < 1e-4
    print("\nall-reduce of 4 MiB on", world, "GPUs:", {k: round(v, 1) for k, v in results[0].items() if k.endswith("_us")},
          "multicast:", results[0]["multicast"])
