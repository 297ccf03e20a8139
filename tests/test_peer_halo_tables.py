# SPDX-License-Identifier: Apache-2.0
"""Pull tables of the peer-memory engine (owner rank, owner row, lattice image per ghost) checked on CPU ranks: emulating
the pull over the gathered owner buffers must reproduce the ghost positions of the send/receive plan, for slabs with
periodic dimensions kept local and for 3-D rank grids."""
import os

import pytest
import torch


def _worker(rank: int, world: int, port: int, grid, q) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        import torch.distributed as dist

        dist.init_process_group("gloo", rank=rank, world_size=world)
        from nvalchemi_toolkit_b200 import Batch
        from nvalchemi_toolkit_b200.distributed import DomainConfig, ShardedBatch
        from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows
        from nvalchemi_toolkit_b200.distributed.peer_halo import build_pull_tables
        from nvalchemi_toolkit_b200.distributed.spec import SPEC_MACE_HALO
        from tests.helpers import fcc_supercell

        b = Batch.from_data_list([fcc_supercell(8, noise=0.08, seed=3)])
        cfg = DomainConfig(cutoff=5.0, skin=1.0, grid_dims=grid)
        sh = ShardedBatch.from_batch(b, cfg, SPEC_MACE_HALO.with_(refresh_per_layer=True), local_periodic=True)
        t = build_pull_tables(sh)
        cell = sh.cell.float()
        own = sh.owned.positions + t["wrap_image"] @ cell      # what each owner keeps in its symmetric buffer
        allbuf, counts = all_gather_rows(own)
        start = torch.cumsum(torch.tensor([0] + counts[:-1]), 0)
        rows_ok = bool((t["home_row"].long() < torch.tensor(counts)[t["home_rank"].long()]).all())
        ghost = allbuf[start[t["home_rank"].long()] + t["home_row"].long()] + t["ghost_image"] @ cell
        ref = sh.halo.forward_positions(sh.owned.positions, sh.cell)
        # reverse path: every owner pulls what the holders accumulated on their copies of its rows
        g = torch.Generator().manual_seed(10 + rank)
        local = torch.randn(sh.n_owned + sh.n_ghost, 4, generator=g)
        every, cnt = all_gather_rows(local)
        base = torch.cumsum(torch.tensor([0] + cnt[:-1]), 0)
        pulled = local[: sh.n_owned].clone()
        pulled.index_add_(0, t["send_row"].long(), every[base[t["send_peer"].long()] + t["send_peer_row"].long()])
        want = sh.halo.reverse_add(local[sh.n_owned:].clone(), local[: sh.n_owned].clone())
        n_ghost_of = torch.tensor([c for c in cnt]) - torch.tensor(counts)
        used_ok = bool((t["send_used_index"].long() < n_ghost_of[t["send_peer"].long()]).all()) and \
            bool((t["send_peer_row"].long() - t["send_used_index"].long() == torch.tensor(counts)[t["send_peer"].long()]).all())
        q.put((rank, {"err": float((ghost - ref).abs().max()), "rows_ok": rows_ok, "ghost": sh.n_ghost,
                      "rev_err": float((pulled - want).abs().max()), "used_ok": used_ok,
                      "local_pbc": sh.halo.local_pbc.tolist()}))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback

        q.put((rank, {"error": f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"}))


@pytest.mark.parametrize("world,grid", [(2, (2, 1, 1)), (2, (1, 1, 2)), (4, (2, 2, 1))])
def test_pull_tables_reproduce_plan_positions(world, grid):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29820 + world + grid[2], grid, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.terminate()
    for r, res in results.items():
        assert "error" not in res, res["error"]
        assert res["rows_ok"] and res["ghost"] > 0 and res["err"] < 1e-5
        assert res["rev_err"] < 1e-5 and res["used_ok"]
        assert res["local_pbc"] == [g == 1 for g in grid]
