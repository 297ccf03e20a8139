# SPDX-License-Identifier: Apache-2.0
"""Bandwidth of the peer-memory halo kernels (``halo_pull_rows``, ``halo_push_add_rows``) and latency of the flag
barrier, timed on the device with CUDA events and reported as the maximum over ranks.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m nvalchemi_toolkit_b200.benchmark.halo_bandwidth

Every rank pulls ``--rows`` ghost rows from each of ``--peers`` other ranks (rows spread with a stride over the owner's
buffer, as boundary atoms are) and returns as many gradient rows, once by remote reductions issued by the holder
(``push_add``) and once by the owner fetching its copies (``pull_add``, the path the MD engine uses).  Row widths: 512 floats (sender features of a
``128x0e+128x1o`` layer) and 3 floats (positions / forces).  The roofline is the bytes that cross NVLink divided by the
per-direction link bandwidth (``--link-gbs``)."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b) / iters], device="cuda", dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=57344, help="ghost rows per rank (all peers together)")
    ap.add_argument("--owned", type=int, default=131072, help="rows every rank owns")
    ap.add_argument("--peers", type=int, default=2, help="number of ranks a rank takes ghosts from")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--single-process", action="store_true",
                    help="one process, one GPU: the peers' buffers are plain allocations of this GPU (the kernels are the same, "
                         "the traffic stays in local memory); for profiler captures of the kernels, not for bandwidth claims")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from nvalchemi_toolkit_b200.ops._native_counter import ops
    from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

    if args.single_process:
        rank, world = 0, 1 + max(1, args.peers)
    else:
        dist.init_process_group("nccl", device_id=dev)
        rank, world = dist.get_rank(), dist.get_world_size()
    peers = max(1, min(args.peers, world - 1))
    g = args.rows // peers * peers
    cap = args.owned + g
    nbytes_arena = 4 * cap * (512 + 512 + 3 + 3) + (1 << 16)
    p2p = P2PContext.single_process(nbytes_arena, dev, world) if args.single_process else P2PContext(nbytes_arena, dev)
    feat, feat_ptrs = p2p.arena.alloc((cap, 512))
    grad, grad_ptrs = p2p.arena.alloc((cap, 512))
    pos, pos_ptrs = p2p.arena.alloc((cap, 3))
    gpos, gpos_ptrs = p2p.arena.alloc((cap, 3))
    feat.normal_()
    pos.normal_()
    per = g // peers
    home_rank = torch.cat([torch.full((per,), (rank + 1 + k) % world, dtype=torch.int32, device=dev) for k in range(peers)])
    stride = max(1, args.owned // per)
    home_row = (torch.arange(per, device=dev, dtype=torch.int32) * stride % args.owned).repeat(peers).contiguous()
    shift = torch.zeros(g, 3, device=dev)
    if not args.single_process:
        p2p.barrier()
    res = {"single_process": bool(args.single_process), "world": world, "ghost_rows": g, "peers": peers, "link_gbs_per_direction": args.link_gbs}
    for name, buf, ptrs, width, sh in (("features_512", feat, feat_ptrs, 512, None), ("positions_3", pos, pos_ptrs, 3, shift)):
        ms = _time(lambda: ops.halo_pull_rows(buf, args.owned, home_rank, home_row, sh, ptrs), args.iters)
        nbytes = g * width * 4
        res[f"pull_{name}"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "of_link": nbytes / ms / 1e6 / args.link_gbs}
    grad[args.owned:].normal_()
    gpos[args.owned:].normal_()
    for name, buf, ptrs, width in (("features_512", grad, grad_ptrs, 512), ("positions_3", gpos, gpos_ptrs, 3)):
        ms = _time(lambda: ops.halo_push_add_rows(buf, args.owned, home_rank, home_row, ptrs), args.iters)
        nbytes = g * width * 4
        res[f"push_add_{name}"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "of_link": nbytes / ms / 1e6 / args.link_gbs}
    # the same gradient rows fetched by their owners instead (plain peer loads + local reductions)
    ghost_row = (args.owned + torch.arange(g, device=dev, dtype=torch.int32)).contiguous()
    for name, buf, ptrs, width in (("features_512", grad, grad_ptrs, 512), ("positions_3", gpos, gpos_ptrs, 3)):
        ms = _time(lambda: ops.halo_pull_add_rows(buf, home_row, home_rank, ghost_row, ptrs), args.iters)
        nbytes = g * width * 4
        res[f"pull_add_{name}"] = {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "of_link": nbytes / ms / 1e6 / args.link_gbs}
    if not args.single_process:  # nobody sets the emulated peers' flags: the barrier is a multi-process measurement
        res["barrier_us"] = 1e3 * _time(p2p.barrier, 200)
    res["status"] = p2p.status()
    if rank == 0:
        print(json.dumps(res))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
