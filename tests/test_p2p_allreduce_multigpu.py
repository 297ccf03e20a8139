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
        # float64 sums through the shared reducer: odd lengths, a scalar, a non-contiguous tensor, a misaligned slice
        from nvalchemi_toolkit_b200.parallel.symmetric import peer_reducer

        red = peer_reducer(None, dev)
        g = torch.Generator(device=dev).manual_seed(7 + rank)
        base = torch.randn(2003, 2, generator=g, device=dev, dtype=torch.float64)
        cases = {"odd": base.clone(), "scalar": base.sum(), "strided": base.t()[:, ::2], "slice": base.reshape(-1)[1:1000]}
        worst = 0.0
        for name, t in cases.items():
            want = t.clone().contiguous()
            dist.all_reduce(want)
            got = red(t if name in ("strided", "slice") else t.clone())  # views: the non-contiguous and the misaligned path
            worst = max(worst, float((got - want).abs().max()))
        res["f64_err"], res["f64_calls"], res["f64_fallbacks"] = worst, red.calls, red.fallbacks
        gathered = [torch.empty_like(base) for _ in range(world)]
        mine = red(base.clone())
        dist.all_gather(gathered, mine)
        res["f64_bitwise_same"] = all(torch.equal(gathered[0], x) for x in gathered)
        sk = torch.randn(4096, 2, device=dev, dtype=torch.float64)
        for fn, key in ((red, "f64_peer_us"), (lambda t: dist.all_reduce(t), "f64_nccl_us")):
            for _ in range(3):
                fn(sk)
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(20):
                fn(sk)
            t1.record()
            torch.cuda.synchronize()
            res[key] = t0.elapsed_time(t1) * 50.0
        res["status"] = max(res["status"], red.ctx.status())
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
        assert res["f64_err"] < 1e-12 and res["f64_calls"] >= 4 and res["f64_fallbacks"] == 0 and res["f64_bitwise_same"]
    print("\nall-reduce of 4 MiB on", world, "GPUs:", {k: round(v, 1) for k, v in results[0].items() if k.endswith("_us")},
          "multicast:", results[0]["multicast"])


def _hook_worker(rank: int, world: int, port: int, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist

        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from nvalchemi_toolkit_b200 import Batch
        from nvalchemi_toolkit_b200.training.hooks import FusedGradAllReduceHook
        from tests.test_training import _dataset, _strategy

        data = _dataset(8)
        hook = FusedGradAllReduceHook(bucket_mb=0.002, status_check="sync")  # ~500 floats per bucket: several buckets
        st = _strategy(num_steps=3, hooks=[hook], devices=[str(dev)])
        for step in range(3):
            lo = 4 * (step % 2) + 2 * rank
            st.train_batch(Batch.from_data_list(data[lo: lo + 2], device=dev))
        torch.cuda.synchronize()
        q.put((rank, {"params": [p.detach().reshape(-1).cpu().tolist() for p in st.models["main"].parameters()],
                      "buckets": len(hook._buckets), "overlapped": hook.num_overlapped, "status": hook._p2p.status()}))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, {"error": f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"}))


def test_bucketed_gradient_allreduce_overlaps_backward_and_matches_single_process():
    """The training hook on 2 GPUs: several buckets, reductions launched from inside backward, parameters identical on
    both ranks and equal to a single-process run on the union of the two ranks' batches."""
    import torch.multiprocessing as mp

    from nvalchemi_toolkit_b200 import Batch
    from tests.test_training import _dataset, _strategy

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hook_worker, args=(r, 2, 29571, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    for r in res.values():
        assert "error" not in r, r["error"]
        assert r["status"] == 0 and r["buckets"] > 1 and r["overlapped"] >= 1
    for a, b in zip(res[0]["params"], res[1]["params"]):
        assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=1e-7)
    data = _dataset(8)
    st = _strategy(num_steps=3)
    for step in range(3):
        st.train_batch(Batch.from_data_list(data[4 * (step % 2): 4 * (step % 2) + 4]))
    for a, b in zip(res[0]["params"], st.models["main"].parameters()):
        assert torch.allclose(torch.tensor(a), b.detach().reshape(-1), atol=5e-3)
