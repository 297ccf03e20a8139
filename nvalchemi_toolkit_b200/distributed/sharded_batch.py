# SPDX-License-Identifier: Apache-2.0
"""``ShardedBatch``: one large system split over ranks by spatial sub-domain.

Reference: ``nvalchemi/distributed/sharded_batch.py:60-930`` (``from_batch``, ``local_batch``, ``padded_batch``,
``gather``/``to_global_batch``, migration).  Each rank holds an ordinary :class:`Batch` with its *owned* atoms (so every
integrator kernel and hook works on it unchanged) plus a :class:`HaloExchange` plan.  The *padded* batch appends ghost
rows and is what the model sees; it is an open-boundary cluster (periodic images are explicit ghost rows), so a model
needs no PBC support to run domain-decomposed.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.distributed.config import DomainConfig
from nvalchemi_toolkit_b200.distributed.halo import HaloExchange, _world, all_gather_rows, migrate_rows
from nvalchemi_toolkit_b200.distributed.partitioner import SpatialPartitioner
from nvalchemi_toolkit_b200.distributed.spec import MLIPSpec

_GHOST_STATIC = ("atomic_numbers", "charges", "node_charges", "atom_categories")


def _node_fields(batch: Batch) -> dict[str, torch.Tensor]:
    g = batch._atoms_group
    return {k: g[k] for k in g.keys()}


def _system_fields(batch: Batch) -> dict[str, torch.Tensor]:
    g = batch._system_group
    return {k: g[k] for k in g.keys()} if g is not None else {}


def _make_batch(node: dict[str, torch.Tensor], system: dict[str, torch.Tensor], template: Batch) -> Batch:
    levels = {k: "node" for k in node}
    levels.update({k: "system" for k in system})
    merged = dict(node)
    merged.update(system)
    return Batch.from_raw_dicts([merged], field_levels=levels, device=node["positions"].device,
                                data_class=template._data_class)


class ShardedBatch:
    def __init__(self, owned: Batch, global_ids: torch.Tensor, n_global: int, partitioner: SpatialPartitioner,
                 config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None,
                 local_periodic: bool = False) -> None:
        if owned.num_graphs != 1:
            raise ValueError("domain decomposition shards ONE system; batch many small systems instead of sharding them")
        self.owned, self.global_ids, self.n_global = owned, global_ids, int(n_global)
        self.partitioner, self.config, self.spec, self.group = partitioner, config, spec, group
        self.rank, self.world = _world(group)
        width = config.ghost_width
        if spec is not None:
            width = max(width, spec.ghost_width(config.cutoff, config.skin)) if spec.message_passes > 0 else 0.0
        if width > 0.0 and self.world > 1:
            width += config.migration_hysteresis  # owned atoms may sit this far outside their owner's box
        self.local_periodic = bool(local_periodic)
        self.halo = HaloExchange(partitioner, width, group, local_periodic=self.local_periodic)
        self._extra_halos: dict[float, HaloExchange] = {}
        self._ref_positions: torch.Tensor | None = None
        self._ghost_static: dict[int, dict[str, torch.Tensor]] = {}
        self.num_migrated = 0
        self._flag_host: torch.Tensor | None = None
        self._flag_event: Any = None
        self._flag_pending = False
        self.rebuild(migrate=False)

    # ---- construction --------------------------------------------------------
    @classmethod
    def from_batch(cls, batch: Batch, config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None,
                   local_periodic: bool = False) -> "ShardedBatch":
        """Every rank passes the same (replicated) single-system batch and keeps the atoms inside its sub-domain."""
        rank, world = _world(group)
        cell = batch.cell.reshape(3, 3)
        pbc = batch.pbc.reshape(3) if getattr(batch, "pbc", None) is not None else torch.zeros(3, dtype=torch.bool)
        part = SpatialPartitioner(cell, pbc, world, config.cutoff + config.skin, grid_dims=config.grid_dims,
                                  hysteresis=config.migration_hysteresis)
        owner = part.assign_atoms_to_ranks(batch.positions)
        mine = torch.nonzero(owner == rank, as_tuple=False).flatten()
        # The assignment is computed from the replicated system, so every rank sees every rank's count and all of them
        # raise together (a rank that raised alone would leave the others waiting in their next collective).
        counts = torch.bincount(owner.reshape(-1).long(), minlength=world)
        empty = torch.nonzero(counts == 0).flatten().tolist()
        if config.require_nondegenerate and empty:
            raise RuntimeError(f"degenerate domain decomposition: rank(s) {empty} of {world} own no atoms of the "
                               f"{batch.num_nodes}-atom system (rank grid {part.grid}); use fewer ranks, a larger system, "
                               "or set require_nondegenerate=False")
        node = {k: v[mine] for k, v in _node_fields(batch).items()}
        owned = _make_batch(node, _system_fields(batch), batch)
        return cls(owned, mine.to(torch.int64), batch.num_nodes, part, config, spec, group, local_periodic=local_periodic)

    # ---- views ---------------------------------------------------------------
    @property
    def n_owned(self) -> int:
        return self.owned.num_nodes

    @property
    def n_ghost(self) -> int:
        return self.halo.n_ghost

    @property
    def local_batch(self) -> Batch:
        return self.owned

    @property
    def cell(self) -> torch.Tensor:
        return self.owned.cell.reshape(3, 3)

    def owned_mask(self) -> torch.Tensor:
        m = torch.zeros(self.n_owned + self.n_ghost, dtype=torch.bool, device=self.owned.device)
        m[: self.n_owned] = True
        return m

    def halo_for(self, ghost_width: float) -> HaloExchange:
        """A ghost plan of its own width over the same owned partition (members of a composite model need different
        halo depths; a short-ranged member should not pay for the deepest one)."""
        width = float(ghost_width)
        if width > 0.0 and self.world > 1:
            width += self.config.migration_hysteresis
        if abs(width - self.halo.width) < 1e-12:
            return self.halo
        if width > self.halo.width:
            raise ValueError("a member halo cannot be wider than the sharded batch's own halo")
        key = round(width, 9)
        if key not in self._extra_halos:
            halo = HaloExchange(self.partitioner, width, self.group, local_periodic=self.local_periodic)
            halo.build(self.owned.positions.detach(), self.global_ids)
            self._extra_halos[key] = halo
            self._ghost_static[id(halo)] = self._static_for(halo)
        return self._extra_halos[key]

    def _static_for(self, halo: HaloExchange) -> dict[str, torch.Tensor]:
        return {k: halo.forward(getattr(self.owned, k)) for k in _GHOST_STATIC
                if getattr(self.owned, k, None) is not None and getattr(self.owned, k).shape[0] == self.n_owned}

    def padded_batch(self, halo: HaloExchange | None = None) -> Batch:
        """Owned rows followed by ghost rows, open boundaries, current positions."""
        halo = halo if halo is not None else self.halo
        pos = self.owned.positions
        allpos = torch.cat([halo.owned_positions(pos, self.cell), halo.forward_positions(pos, self.cell)])
        node = {"positions": allpos}
        for k, ghost in self._ghost_static[id(halo)].items():
            node[k] = torch.cat([getattr(self.owned, k), ghost])
        system = {k: v for k, v in _system_fields(self.owned).items() if k in ("cell", "total_charge", "spin")}
        system["pbc"] = halo.local_pbc.reshape(1, 3).to(pos.device)
        weights = torch.zeros(allpos.shape[0], dtype=pos.dtype, device=pos.device)
        weights[: self.n_owned] = 1.0
        node["energy_weights"] = weights
        padded = _make_batch(node, system, self.owned)
        object.__setattr__(padded, "_dd", (self.group, self.world))  # models with global sums reduce over this group
        return padded

    # ---- maintenance ---------------------------------------------------------
    def needs_rebuild(self) -> bool:
        """True on every rank if any atom anywhere moved more than half the skin since the last rebuild."""
        if self._ref_positions is None or self._ref_positions.shape != self.owned.positions.shape:
            moved = torch.ones((), device=self.owned.device)
        elif self.config.skin <= 0.0:
            moved = torch.ones((), device=self.owned.device)
        else:
            d2 = (self.owned.positions.detach() - self._ref_positions).pow(2).sum(-1)
            lim = (0.5 * self.config.skin) ** 2
            moved = (d2.max() > lim).to(torch.float32) if d2.numel() else torch.zeros((), device=self.owned.device)
        if self.world > 1:
            moved = moved.to(torch.float32)
            dist.all_reduce(moved, op=dist.ReduceOp.MAX, group=self.group)
        return bool(moved > 0)

    # ---- asynchronous consensus (no step waits for the flag it raises) ---------
    def dispatch_rebuild_check(self) -> None:
        """Start the "has any atom anywhere moved more than skin / 2" reduction for the CURRENT positions; the answer
        is read by :meth:`consume_rebuild_check` at the next step.  Reference:
        ``nvalchemi/distributed/strategy.py:320-344`` (asynchronous all-reduce consumed one step later).

        The flag trails the positions by one step: the forces of the step that raised it were evaluated with the old
        ghost lists.  That is exact as long as two consecutive steps move no atom further than the remaining half of the
        skin; keep ``skin`` above four times the largest per-step displacement."""
        pos = self.owned.positions.detach()
        if self._ref_positions is None or self._ref_positions.shape != pos.shape or self.config.skin <= 0.0:
            flag = torch.ones(1, dtype=torch.int32, device=pos.device)
        else:
            d2 = (pos - self._ref_positions).pow(2).sum(-1)
            lim = (0.5 * self.config.skin) ** 2
            flag = (d2.max() > lim).to(torch.int32).reshape(1) if d2.numel() else torch.zeros(1, dtype=torch.int32, device=pos.device)
        if self.world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if pos.is_cuda:
            if self._flag_host is None:
                self._flag_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._flag_host.copy_(flag, non_blocking=True)
            self._flag_event = torch.cuda.Event()
            self._flag_event.record()
        else:
            self._flag_host = flag.clone()
            self._flag_event = None
        self._flag_pending = True

    def consume_rebuild_check(self) -> bool:
        """Result of the last :meth:`dispatch_rebuild_check` (False when none is pending)."""
        if not self._flag_pending:
            return False
        self._flag_pending = False
        if self._flag_event is not None:
            self._flag_event.synchronize()
        return bool(int(self._flag_host[0]))

    def rebuild(self, migrate: bool = True) -> None:
        """Re-derive ownership (with hysteresis), move rows that changed owner, and rebuild the ghost plan."""
        self.partitioner.update_cell(self.cell)  # barostats change the cell; fractional boxes stay as they are
        if migrate and self.world > 1:
            pos = self.owned.positions.detach()
            here = torch.full((self.n_owned,), self.rank, dtype=torch.long, device=pos.device)
            keep = self.partitioner.keeps_owner(pos, here)
            new_owner = torch.where(keep, here, self.partitioner.assign_atoms_to_ranks(pos))
            moved = int((new_owner != self.rank).sum())
            total = torch.tensor([moved], device=pos.device)
            dist.all_reduce(total, group=self.group)
            if int(total) > 0:
                fields = _node_fields(self.owned)
                fields["__gid"] = self.global_ids
                fields = migrate_rows({k: v.detach() for k, v in fields.items()}, new_owner, self.group)
                self.global_ids = fields.pop("__gid")
                self.owned = _make_batch(fields, _system_fields(self.owned), self.owned)
                self.num_migrated += int(total)
        self.halo.build(self.owned.positions.detach(), self.global_ids)
        self._ghost_static = {id(self.halo): self._static_for(self.halo)}
        for halo in self._extra_halos.values():
            halo.build(self.owned.positions.detach(), self.global_ids)
            self._ghost_static[id(halo)] = self._static_for(halo)
        self._ref_positions = self.owned.positions.detach().clone()
        self._flag_pending = False

    # ---- gathering -----------------------------------------------------------
    def gather(self, dst: int | None = None) -> Batch | None:
        """The global batch in original atom order (on ``dst`` only, or on every rank when ``dst`` is None)."""
        if self.world == 1:
            order = torch.argsort(self.global_ids)
            node = {k: v[order] for k, v in _node_fields(self.owned).items()}
            return _make_batch(node, _system_fields(self.owned), self.owned)
        fields = _node_fields(self.owned)
        fields["__gid"] = self.global_ids
        out: dict[str, torch.Tensor] = {}
        for k in sorted(fields):
            out[k], _ = all_gather_rows(fields[k].detach().contiguous(), self.group)
        if dst is not None and self.rank != dst:
            return None
        order = torch.argsort(out.pop("__gid"))
        return _make_batch({k: v[order] for k, v in out.items()}, _system_fields(self.owned), self.owned)

    to_global_batch = gather
