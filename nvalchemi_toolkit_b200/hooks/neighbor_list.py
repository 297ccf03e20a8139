# SPDX-License-Identifier: Apache-2.0
"""``NeighborListHook``: keeps the batch's neighbour data current during dynamics.

Reference behaviour (``nvalchemi/hooks/neighbor_list.py:112-760``): build at ``BEFORE_COMPUTE``; with a Verlet
``skin`` the list is built for ``cutoff + skin`` and rebuilt only for systems in which some atom moved more
than ``skin / 2`` since the last build (minimum image); the matrix width ``K`` adapts: an overflow grows it by
1.5x (rounded to 16) and triggers a rebuild.  Rebuild detection and the cell-list search are device kernels;
the only host synchronisation is the overflow check after a (rare) rebuild.
"""
from __future__ import annotations

from enum import Enum
from typing import Any

import torch

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.models.base import NeighborConfig, NeighborListFormat


class NeighborListHook:
    def __init__(self, config: NeighborConfig, skin: float = 0.0, max_neighbors: int | None = None,
                 stage: Enum | None = None, method: str | None = None) -> None:
        self.config = config
        self.skin = float(skin)
        self.stage = stage
        if method not in (None, "auto", "cell_list", "naive"):
            raise ValueError(f"unknown neighbour-list method {method!r}; expected 'auto', 'cell_list' or 'naive'")
        #: "cell_list" (binned search kernel, any size), "naive" (all pairs with periodic images, plain tensor
        #: expressions: only sensible for systems of a few hundred atoms) or "auto" / None (cell list)
        self.method = method
        #: shrink the matrix width again when the largest count has stayed below half of it for this many rebuilds
        self.shrink_after = 8
        self._low_use = 0
        self.frequency = 1
        self._max_neighbors = max_neighbors
        self._ref_positions: torch.Tensor | None = None
        self._flags: torch.Tensor | None = None
        self._bufs: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None
        self._shape_key: tuple | None = None
        self.num_rebuilds = 0
        self.version = 0  # incremented on every rebuild; consumers cache derived edge lists against it

    def _alloc(self, batch: Any, k: int) -> None:
        n, dev = batch.num_nodes, batch.device
        self._bufs = (torch.full((n, k), n, dtype=torch.int32, device=dev),
                      torch.zeros(n, dtype=torch.int32, device=dev),
                      torch.zeros(n, k, 3, dtype=torch.int32, device=dev))

    def _build(self, batch: Any, cell: torch.Tensor, pbc: torch.Tensor, flags: torch.Tensor | None) -> None:
        cutoff = self.config.cutoff + self.skin
        k = self._bufs[0].shape[1]
        while True:
            if self.method == "naive":
                _nb._neighbor_matrix_torch(batch.positions.detach(), cell, pbc, batch.batch_idx, cutoff, *self._bufs,
                                           self.config.half_list)
            else:
                _nb.neighbor_matrix(batch.positions, cell, pbc, batch.batch_idx, batch.batch_ptr, cutoff, k,
                                    self.config.half_list, out=self._bufs, rebuild_flags=flags)
            actual = int(self._bufs[1].max())
            if actual <= k:
                break
            k = ((int(actual * 1.5) + 1) + 15) // 16 * 16
            self._alloc(batch, k)
            flags = None  # a wider matrix needs every row rebuilt
        # adaptive shrink: a width that has been more than twice the need for a while costs memory and bandwidth
        self._low_use = self._low_use + 1 if (self._max_neighbors is None and actual * 2 < k and k > 16) else 0
        if self._low_use >= self.shrink_after:
            k_new = max(16, ((int(actual * 1.25) + 1) + 15) // 16 * 16)
            if k_new < k:
                self._alloc(batch, k_new)
                _nb.neighbor_matrix(batch.positions, cell, pbc, batch.batch_idx, batch.batch_ptr, cutoff, k_new,
                                    self.config.half_list, out=self._bufs)
            self._low_use = 0
        self.num_rebuilds += 1
        self.version += 1

    def __call__(self, ctx: Any, stage: Enum) -> None:
        batch = ctx.batch
        cell, pbc = _nb.cell_and_pbc(batch)
        key = (batch.num_nodes, batch.num_graphs, batch.device, batch.positions.dtype)
        fresh = self._bufs is None or key != self._shape_key
        if not fresh:
            # same CSR pointer OBJECT, not written since (tensor version counter): the segmentation is unchanged and no
            # device comparison (= host synchronisation) is needed; only a different or modified tensor is compared
            ptr = batch.batch_ptr
            seen = getattr(self, "_batch_ptr_seen", None)
            if seen is None or seen[0] is not ptr or seen[1] != ptr._version:
                fresh = not torch.equal(self._batch_ptr, ptr)
                self._batch_ptr_seen = (ptr, ptr._version)
        if fresh:
            k = self._max_neighbors
            if k is None:
                k = _nb.estimate_max_neighbors(self.config.cutoff + self.skin)
                if not bool(pbc.any()) and batch.max_num_nodes > 0:
                    k = min(k, (batch.max_num_nodes + 15) // 16 * 16)
            self._shape_key = key
            self._batch_ptr = batch.batch_ptr.clone()
            self._batch_ptr_seen = (batch.batch_ptr, batch.batch_ptr._version)
            self._alloc(batch, k)
            self._build(batch, cell, pbc, None)
            if self.skin > 0.0:
                self._ref_positions = batch.positions.detach().clone()
                self._flags = torch.zeros(batch.num_graphs, dtype=torch.bool, device=batch.device)
        elif self.skin > 0.0:
            self._flags.zero_()
            _ops.batch_neighbor_list_rebuild_inplace(self._ref_positions, batch.positions.detach(), batch.batch_idx,
                                                     self._flags, 0.5 * self.skin, True, cell, torch.linalg.inv(cell), pbc)
            if bool(self._flags.any()):
                self._build(batch, cell, pbc, self._flags)
        else:
            self._build(batch, cell, pbc, None)
        nm, num, sh = self._bufs
        _nb.write_neighbor_data_to_batch(batch, nm, num, sh, self.config.format, self.config.cutoff + self.skin)
        object.__setattr__(batch, "_neighbor_version", (id(self), self.version))
