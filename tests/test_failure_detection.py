# SPDX-License-Identifier: Apache-2.0
"""Failure detection on the host (gloo ranks) and a bounded device-side wait (one GPU, a flag nothing sets)."""
import os
import time

import pytest
import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.distributed.failure import HeartbeatMonitor, PeerFailure, guarded_run


def _worker(rank, world, port, q, mode):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mon = HeartbeatMonitor.from_env(timeout=2.0)
        dist.barrier()
        state = {"steps": 0}

        def pre_step(i):  # local health checks run before the rank declares itself ready for the step
            if rank == 1 and i == 3:
                if mode == "raise":
                    raise ValueError("rank 1 breaks at step 3")
                time.sleep(6.0)  # stall: no readiness message, peers give up on this rank

        def step(i):
            t = torch.ones(1)
            dist.all_reduce(t)  # only reached while every rank is alive
            state["steps"] += 1

        seen = []
        try:
            done = guarded_run(step, 6, mon, pre_step=pre_step, on_failure=seen.append)
            q.put((rank, "stopped", done, [e.ranks for e in seen]))
        except ValueError as exc:
            q.put((rank, "raised", state["steps"], str(exc)))
    finally:
        if mode == "stall" and rank == 1:
            os._exit(0)  # peers are gone; do not wait for them in destroy_process_group
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["raise", "stall"])
def test_peer_failure_is_seen_on_the_host_before_the_next_collective(mode):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 3, 29820 + (mode == "stall"), q, mode)) for r in range(3)]
    for p in procs:
        p.start()
    want = 3 if mode == "raise" else 2
    res = {}
    for _ in range(want):
        item = q.get(timeout=60)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    for r in (0, 2):
        kind, done, failures = res[r]
        assert kind == "stopped" and failures == [[1]]
        assert done == 3  # steps 0-2 ran everywhere; nobody entered the collective of step 3
    if mode == "raise":
        assert res[1][0] == "raised" and "breaks at step 3" in res[1][2]


def test_monitor_with_a_plain_store():
    store = dist.HashStore()
    a = HeartbeatMonitor(store, 0, 2, timeout=0.2)
    b = HeartbeatMonitor(store, 1, 2, timeout=0.2)
    a.beat(2)
    b.beat(2)
    a.check(2)
    with pytest.raises(PeerFailure) as info:
        a.check(3)
    assert info.value.ranks == [1]
    b.fail("out of memory")
    with pytest.raises(PeerFailure, match="announced"):
        a.check(1)


@pytest.mark.gpu
def test_device_barrier_wait_is_bounded_and_reports_status():
    """A two-rank flag barrier whose second rank never arrives: the kernel returns after its bounded wait and sets the
    status word; the context stays usable."""
    dev = torch.device("cuda", 0)
    flags = torch.zeros(2, 64, dtype=torch.int32, device=dev)  # row r = flag row of rank r; row 1 is never written by a peer
    ptrs = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.time()
    torch.ops.nvalchemi.p2p_barrier(ptrs, 0, 2, 1, err)
    torch.cuda.synchronize()
    assert 0.2 < time.time() - t0 < 20.0
    assert int(err) == 101  # 100 + the rank that did not arrive
    x = torch.ones(8, device=dev) * 2
    assert float(x.sum()) == 16.0  # the context is alive


@pytest.mark.gpu
def test_allreduce_reports_a_peer_that_never_arrives():
    """``P2PContext.allreduce_`` over a context whose second "rank" is a plain buffer nothing drives: both rendezvous
    run into their bounded wait, the call returns, and the status check raises instead of handing out a sum of
    incomplete buffers (immediately with ``check="sync"``, at the following call with ``check="lazy"``)."""
    from nvalchemi_toolkit_b200.distributed.failure import PeerFailure
    from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

    dev = torch.device("cuda", 0)
    ctx = P2PContext.single_process(4096, dev, world=2)
    view, _ = ctx.arena.alloc((256,), torch.float32)
    view.fill_(1.0)
    out = torch.empty_like(view)
    with pytest.raises(PeerFailure) as info:
        ctx.allreduce_(view, 0.5, out=out, use_multimem=False, check="sync")
    assert info.value.ranks == [1]
    lazy = P2PContext.single_process(4096, dev, world=2)
    v2, _ = lazy.arena.alloc((256,), torch.float32)
    lazy.allreduce_(v2, 1.0, out=out, use_multimem=False, check="lazy")  # returns: the failure is only posted
    torch.cuda.synchronize()
    with pytest.raises(PeerFailure):
        lazy.allreduce_(v2, 1.0, out=out, use_multimem=False, check="lazy")
    assert float((torch.ones(4, device=dev) * 3).sum()) == 12.0  # the context is alive
