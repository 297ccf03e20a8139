# SPDX-License-Identifier: Apache-2.0
"""Graph (node) partition: every rank owns a contiguous INDEX block of the atoms and evaluates only the edges whose
receiver it owns; the sender rows it needs from other blocks are exchanged before every message-passing layer and the
gradients that land on them are returned to their owners.

Reference: ``nvalchemi/distributed/strategy.py:442-499,543-677`` and ``distributed/distributed_model.py:394-430,1061-1077``
(balanced node blocks, per-layer feature all-gather with a reduce-scatter adjoint, ``reduce_scatter_tensor`` for
forces).  Differences: instead of gathering ALL node rows on every rank each layer, a rank requests only the rows its own
edges reference (found from a neighbour search over the gathered geometry with rows for its own block only), so the
per-layer traffic is the one-hop boundary of the block, and forces come back by the reverse of the same exchange.  No
spatial locality is assumed: the partition works for clusters, molecules and arbitrarily ordered atoms (with spatially
sorted atoms it degenerates into a slab decomposition).

:class:`GraphHalo` exposes the interface of :class:`HaloExchange`, and :class:`GraphShardedBatch` that of
:class:`ShardedBatch`, so ``DistributedModel``, ``HaloDispatchMode`` (per-layer refresh of unmodified models) and
``DomainParallel`` run on them unchanged: ``DomainConfig(strategy="graph_partition")`` selects this module.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.distributed.config import DomainConfig
from nvalchemi_toolkit_b200.distributed.halo import HaloExchange, _world, all_gather_rows, all_to_all_rows, exchange_counts
from nvalchemi_toolkit_b200.distributed.partitioner import IndexPartitioner
from nvalchemi_toolkit_b200.distributed.sharded_batch import ShardedBatch, _make_batch, _node_fields, _system_fields
from nvalchemi_toolkit_b200.distributed.spec import MLIPSpec


class GraphHalo(HaloExchange):
    """Ghost rows chosen by connectivity: the atoms of other blocks within ``reach`` of an owned atom."""

    def __init__(self, partitioner: IndexPartitioner, reach: float, pbc: torch.Tensor, group: Any = None) -> None:
        self.index_part, self.width, self.group = partitioner, float(reach), group
        self.part = None
        self.rank, self.world = _world(group)
        self.local_periodic = True
        self._pbc = pbc.reshape(3).bool().cpu()
        self.send_index = self.send_shift = self.wrap_shift = None
        self.send_splits, self.recv_splits = [], []
        self.ghost_global_id = self.ghost_owner_rank = None
        self.num_builds = 0
        self.edges_owned = 0

    @property
    def local_pbc(self) -> torch.Tensor:
        return self._pbc.clone()  # periodic images are applied by the neighbour search, never unrolled into rows

    def build(self, positions: torch.Tensor, global_ids: torch.Tensor, cell: torch.Tensor | None = None) -> None:
        """``positions`` / ``global_ids``: the rank's owned block.  Gathers the geometry, finds the senders its rows
        need, and negotiates the send lists (one request exchange; geometry is gathered only here, at list rebuilds)."""
        dev = positions.device
        lo, hi = self.index_part.block(self.rank)
        n_own = hi - lo
        all_pos, counts = all_gather_rows(positions.detach().contiguous(), self.group)
        n_all = all_pos.shape[0]
        # this rank's block first, so that the neighbour search can stop after the owned rows
        order = torch.cat([torch.arange(lo, hi, device=dev), torch.arange(0, lo, device=dev), torch.arange(hi, n_all, device=dev)])
        cellb = (cell if cell is not None else torch.eye(3, dtype=positions.dtype, device=dev)).reshape(1, 3, 3).to(positions.dtype)
        k = _nb.estimate_max_neighbors(self.width)
        b_idx = torch.zeros(n_all, dtype=torch.int32, device=dev)
        b_ptr = torch.tensor([0, n_all], dtype=torch.int32, device=dev)
        while True:
            nm = torch.full((max(n_own, 1), k), n_all, dtype=torch.int32, device=dev)
            num = torch.zeros(max(n_own, 1), dtype=torch.int32, device=dev)
            sh = torch.zeros(max(n_own, 1), k, 3, dtype=torch.int32, device=dev)
            if n_own:
                _nb.neighbor_matrix(all_pos[order].contiguous(), cellb.contiguous(), self._pbc.reshape(1, 3).to(dev), b_idx, b_ptr,
                                    self.width, k, False, out=(nm, num, sh), num_rows=n_own)
            mx = int(num.max()) if n_own else 0
            if mx <= k:
                break
            k = ((int(mx * 1.5) + 1) + 15) // 16 * 16
        valid = torch.arange(k, device=dev)[None, :] < num[:, None]
        self.edges_owned = int(valid.sum()) if n_own else 0
        senders = order[nm[valid].long()] if n_own else order[:0]       # global ids
        need = torch.unique(senders[(senders < lo) | (senders >= hi)])  # sorted: grouped by owner block
        owner = self.index_part.owner(need)
        want_counts = torch.bincount(owner, minlength=self.world).tolist()
        self.recv_splits = [int(c) for c in want_counts]
        # tell every owner which of its rows this rank wants
        give_counts = exchange_counts(self.recv_splits, dev, self.group) if self.world > 1 else list(self.recv_splits)
        requested = all_to_all_rows(need, self.recv_splits, give_counts, self.group)
        self.send_splits = [int(c) for c in give_counts]
        self.send_index = (requested - lo).long()
        self.send_shift = torch.zeros(self.send_index.numel(), 3, dtype=torch.int32, device=dev)
        self.wrap_shift = torch.zeros(n_own, 3, dtype=torch.int32, device=dev)
        self.ghost_global_id = need
        self.ghost_owner_rank = owner
        self.num_builds += 1

    def forward_positions(self, positions: torch.Tensor, cell: torch.Tensor) -> torch.Tensor:
        return self.forward(positions)

    def owned_positions(self, positions: torch.Tensor, cell: torch.Tensor) -> torch.Tensor:
        return positions


class GraphShardedBatch(ShardedBatch):
    """One system split into contiguous index blocks; same interface as :class:`ShardedBatch`."""

    def __init__(self, owned: Batch, global_ids: torch.Tensor, n_global: int, partitioner: IndexPartitioner,
                 config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None) -> None:
        if owned.num_graphs != 1:
            raise ValueError("graph partition shards ONE system")
        self.owned, self.global_ids, self.n_global = owned, global_ids, int(n_global)
        self.partitioner, self.config, self.spec, self.group = partitioner, config, spec, group
        self.rank, self.world = _world(group)
        self.local_periodic = True
        pbc = owned.pbc.reshape(3) if getattr(owned, "pbc", None) is not None else torch.zeros(3, dtype=torch.bool)
        self.halo = GraphHalo(partitioner, config.cutoff + config.skin, pbc, group)
        self._extra_halos: dict[float, HaloExchange] = {}
        self._ref_positions = None
        self._ghost_static: dict[int, dict[str, torch.Tensor]] = {}
        self.num_migrated = 0
        self._flag_host = None
        self._flag_event = None
        self._flag_pending = False
        self.rebuild(migrate=False)

    @classmethod
    def from_batch(cls, batch: Batch, config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None,
                   local_periodic: bool = True) -> "GraphShardedBatch":
        """Every rank passes the same (replicated) single-system batch and keeps its index block."""
        rank, world = _world(group)
        part = IndexPartitioner(batch.num_nodes, world)
        lo, hi = part.block(rank)
        node = {k: v[lo:hi] for k, v in _node_fields(batch).items()}
        owned = _make_batch(node, _system_fields(batch), batch)
        gids = torch.arange(lo, hi, dtype=torch.int64, device=batch.device)
        return cls(owned, gids, batch.num_nodes, part, config, spec, group)

    def halo_for(self, ghost_width: float) -> HaloExchange:
        return self.halo  # one connectivity-derived ghost set serves every member

    def rebuild(self, migrate: bool = True) -> None:
        """Index ownership never changes; only the ghost lists follow the geometry."""
        self.halo.build(self.owned.positions.detach(), self.global_ids, self.cell)
        self._ghost_static = {id(self.halo): self._static_for(self.halo)}
        self._ref_positions = self.owned.positions.detach().clone()
        self._flag_pending = False
