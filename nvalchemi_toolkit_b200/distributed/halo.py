# SPDX-License-Identifier: Apache-2.0
"""Ghost-atom (halo) exchange over ``torch.distributed`` for any backend (NCCL on GPUs, gloo on CPU).

Reference: ``nvalchemi/distributed/_core/halo_index.py``, ``_core/gather.py``, ``_core/collectives.py`` and
``ops.py:110-540`` (halo forward, backward fold, scatter correction).  Design here: a *plan* is rebuilt rarely (when
the neighbour skin is exhausted) and records, per destination rank, which owned rows are sent and with which integer
lattice shift; between rebuilds a refresh is one variable-size all-to-all of positions, and the reverse exchange adds
ghost-row gradients into their owners.  The peer-memory engine (``distributed/peer_halo.py``) derives its pull tables
from the same plan and then moves rows with NVLink kernels instead of collectives.
"""
from __future__ import annotations

import itertools
import math
import os
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.distributed.partitioner import SpatialPartitioner


def _world(group: Any) -> tuple[int, int]:
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


#: how variable-size row exchanges travel: ``"all_to_all"`` (one ``all_to_all_single`` over the whole group) or ``"p2p"``
#: (``batch_isend_irecv`` with the ranks that actually exchange rows: at most 26 neighbours under a spatial
#: decomposition, however large the group is).  Reference: ``nvalchemi/distributed/_core/collectives.py`` (funcol
#: all-to-all, neighbour-only P2P, gloo isend/irecv fallback).
TRANSPORT = os.environ.get("NVA_HALO_TRANSPORT", "all_to_all")


def neighbor_exchange_rows(rows: torch.Tensor, in_splits: list[int], out_splits: list[int], group: Any = None) -> torch.Tensor:
    """The same result as :func:`all_to_all_rows`, moved with point-to-point messages between the ranks whose split is
    non-empty.  Every rank of the group must call it (peers post the matching receives)."""
    rank, world = _world(group)
    if world == 1:
        return rows
    rows = rows.contiguous()
    out = rows.new_empty((sum(out_splits),) + tuple(rows.shape[1:]))
    ops, so, ro = [], 0, 0
    for peer in range(world):
        ns, nr = in_splits[peer], out_splits[peer]
        if peer == rank:
            if ns:
                out[ro: ro + nr] = rows[so: so + ns]
        else:
            g = dist.get_global_rank(group, peer) if group is not None else peer
            if ns:
                ops.append(dist.P2POp(dist.isend, rows[so: so + ns], g, group))
            if nr:
                ops.append(dist.P2POp(dist.irecv, out[ro: ro + nr], g, group))
        so, ro = so + ns, ro + nr
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out


def all_to_all_rows(rows: torch.Tensor, in_splits: list[int], out_splits: list[int], group: Any = None) -> torch.Tensor:
    """Variable-size all-to-all along dim 0 (identity for a single rank)."""
    _, world = _world(group)
    if world == 1:
        return rows
    if TRANSPORT == "p2p":
        return neighbor_exchange_rows(rows, in_splits, out_splits, group)
    out = rows.new_empty((sum(out_splits),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), out_splits, in_splits, group=group)
    return out


def exchange_counts(counts: list[int], device: torch.device, group: Any = None) -> list[int]:
    _, world = _world(group)
    if world == 1:
        return list(counts)
    send = torch.tensor(counts, dtype=torch.int64, device=device)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.tolist()


def all_gather_rows(rows: torch.Tensor, group: Any = None) -> tuple[torch.Tensor, list[int]]:
    """Concatenation of every rank's rows (ranks may hold different counts) and the per-rank counts."""
    _, world = _world(group)
    if world == 1:
        return rows, [int(rows.shape[0])]
    dev = rows.device
    n = torch.tensor([rows.shape[0]], dtype=torch.int64, device=dev)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n, group=group)
    counts = [int(c) for c in counts]
    m = max(counts)
    padded = rows.new_zeros((m,) + tuple(rows.shape[1:]))
    padded[: rows.shape[0]] = rows
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:c] for p, c in zip(parts, counts)]), counts


class HaloExchange:
    """Send/receive plan for the ghosts of one rank.

    After :meth:`build`, ``n_ghost`` rows arrive ordered by source rank; ``ghost_owner_rank`` and ``ghost_global_id``
    describe them.  ``wrap_shift`` (integer lattice vector per owned atom) maps owned positions into the primary cell
    so that owned and ghost rows live in one consistent frame."""

    def __init__(self, partitioner: SpatialPartitioner, ghost_width: float, group: Any = None,
                 local_periodic: bool = False) -> None:
        self.part, self.width, self.group = partitioner, float(ghost_width), group
        self.rank, self.world = _world(group)
        #: periodic dimensions that the rank grid does not cut keep their periodicity in the local cluster (the
        #: neighbour search applies the images) instead of being unrolled into explicit ghost rows
        self.local_periodic = bool(local_periodic)
        self.send_index: torch.Tensor | None = None
        self.send_shift: torch.Tensor | None = None
        self.send_splits: list[int] = []
        self.recv_splits: list[int] = []
        self.wrap_shift: torch.Tensor | None = None
        self.ghost_global_id: torch.Tensor | None = None
        self.ghost_owner_rank: torch.Tensor | None = None
        self.num_builds = 0

    @property
    def n_ghost(self) -> int:
        return sum(self.recv_splits)

    @property
    def local_pbc(self) -> torch.Tensor:
        """``bool[3]``: dimensions in which the owned + ghost cluster is still periodic."""
        part = self.part
        return torch.tensor([self.local_periodic and bool(part.pbc[d]) and part.grid[d] == 1 for d in range(3)])

    def build(self, positions: torch.Tensor, global_ids: torch.Tensor) -> None:
        part, dev = self.part, positions.device
        f_raw = part.fractional(positions)
        pbc = part.pbc.to(dev)
        # map every owned atom to the periodic image nearest to this rank's box (atoms inside the hysteresis band may
        # sit slightly outside the box, possibly across a periodic face)
        lo_me, hi_me = part.box(self.rank)
        centre = (0.5 * (lo_me + hi_me)).to(dev)
        wrap = torch.where(pbc, -torch.round(f_raw - centre), torch.zeros_like(f_raw))
        f = f_raw + wrap
        self.wrap_shift = wrap.to(torch.int32)
        w = [self.width / part.face[d] for d in range(3)]
        rng = []
        keep = self.local_pbc
        for d in range(3):
            if not bool(part.pbc[d]) or f.shape[0] == 0 or bool(keep[d]):
                rng.append(range(0, 1))
                continue
            fmin, fmax = float(f[:, d].min()), float(f[:, d].max())
            rng.append(range(int(math.floor(-w[d] - fmax)), int(math.ceil(1.0 + w[d] - fmin)) + 1))
        shifts = list(itertools.product(*rng))
        idx_parts, shift_parts, counts = [], [], []
        wt = torch.tensor(w, dtype=torch.float64, device=dev)
        for r in range(self.world):
            lo, hi = part.box(r)
            lo, hi = lo.to(dev) - wt, hi.to(dev) + wt
            # open dimensions: the outermost boxes extend to infinity (atoms may drift past the nominal cell)
            c = part.rank_coords(r)
            for d in range(3):
                if not bool(part.pbc[d]):
                    if c[d] == 0:
                        lo[d] = -float("inf")
                    if c[d] == part.grid[d] - 1:
                        hi[d] = float("inf")
            r_idx, r_shift = [], []
            for s in shifts:
                if r == self.rank and s == (0, 0, 0):
                    continue
                st = torch.tensor(s, dtype=torch.float64, device=dev)
                fs = f + st
                m = ((fs >= lo) & (fs < hi)).all(dim=-1)
                sel = torch.nonzero(m, as_tuple=False).flatten()
                if sel.numel():
                    r_idx.append(sel)
                    r_shift.append((self.wrap_shift[sel] + torch.tensor(s, dtype=torch.int32, device=dev)))
            if r_idx:
                idx_parts.append(torch.cat(r_idx))
                shift_parts.append(torch.cat(r_shift))
                counts.append(int(idx_parts[-1].numel()))
            else:
                counts.append(0)
        self.send_index = torch.cat(idx_parts) if idx_parts else torch.zeros(0, dtype=torch.long, device=dev)
        self.send_shift = torch.cat(shift_parts) if shift_parts else torch.zeros(0, 3, dtype=torch.int32, device=dev)
        self.send_splits = counts
        self.recv_splits = exchange_counts(counts, dev, self.group)
        if self.world == 1:
            self.recv_splits = list(counts)
        self.ghost_global_id = self.forward(global_ids)
        self.ghost_owner_rank = torch.repeat_interleave(
            torch.arange(self.world, device=dev), torch.tensor(self.recv_splits, device=dev))
        self.num_builds += 1

    # ---- per-step traffic ---------------------------------------------------
    def forward(self, owned_rows: torch.Tensor) -> torch.Tensor:
        """Ghost rows of a node-level tensor (owners send ``owned_rows[send_index]``)."""
        return all_to_all_rows(owned_rows[self.send_index], self.send_splits, self.recv_splits, self.group)

    def forward_packed(self, send_rows: torch.Tensor) -> torch.Tensor:
        """Ghost rows from rows that are already in send order (one per entry of ``send_index``)."""
        return all_to_all_rows(send_rows, self.send_splits, self.recv_splits, self.group)

    def reverse_packed(self, ghost_rows: torch.Tensor) -> torch.Tensor:
        """One row per ghost travels back to the rank that sent it; the result is in send order (one row per entry of
        ``send_index``).  No accumulation: use :meth:`reverse_add` for that."""
        return all_to_all_rows(ghost_rows, self.recv_splits, self.send_splits, self.group)

    def forward_positions(self, positions: torch.Tensor, cell: torch.Tensor) -> torch.Tensor:
        """Ghost positions: owner positions plus the recorded lattice shift."""
        shifted = positions[self.send_index] + self.send_shift.to(positions.dtype) @ cell.reshape(3, 3).to(positions.dtype)
        return all_to_all_rows(shifted, self.send_splits, self.recv_splits, self.group)

    def owned_positions(self, positions: torch.Tensor, cell: torch.Tensor) -> torch.Tensor:
        """Owned positions mapped into the frame the ghosts were generated in."""
        return positions + self.wrap_shift.to(positions.dtype) @ cell.reshape(3, 3).to(positions.dtype)

    def reverse_add(self, ghost_rows: torch.Tensor, owned_rows: torch.Tensor) -> torch.Tensor:
        """Add per-ghost contributions (e.g. force on a ghost) into the owners' rows, in place."""
        back = all_to_all_rows(ghost_rows, self.recv_splits, self.send_splits, self.group)
        if back.numel():
            owned_rows.index_add_(0, self.send_index, back.to(owned_rows.dtype))
        return owned_rows


def migrate_rows(fields: dict[str, torch.Tensor], new_owner: torch.Tensor, group: Any = None
                 ) -> dict[str, torch.Tensor]:
    """Move node-level rows to their new owner ranks; returns the rows this rank now owns (stayers first is NOT
    guaranteed; the order is by source rank, which every field shares)."""
    rank, world = _world(group)
    if world == 1:
        return fields
    dev = new_owner.device
    order = torch.argsort(new_owner, stable=True)
    counts = torch.bincount(new_owner, minlength=world).tolist()
    recv = exchange_counts(counts, dev, group)
    return {k: all_to_all_rows(v[order], counts, recv, group) for k, v in fields.items()}
