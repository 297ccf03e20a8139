# SPDX-License-Identifier: Apache-2.0
"""What model code can ask about the decomposition it runs under.

Reference: ``nvalchemi/distributed/_core/context.py`` (``DistributedContext`` in a context variable, ``NOT_DISTRIBUTED``)
and ``_core/routing.py`` (``ShardRouting.from_assignment``: global id ↔ owner rank / local index tables)."""
from __future__ import annotations

import contextlib
import contextvars
from dataclasses import dataclass
from typing import Any, Iterator

import torch


@dataclass(frozen=True)
class DistributedContext:
    rank: int = 0
    world_size: int = 1
    n_owned: int = 0
    n_padded: int = 0
    is_halo: bool = False
    is_sharded: bool = False
    group: Any = None

    @property
    def n_ghost(self) -> int:
        return self.n_padded - self.n_owned


NOT_DISTRIBUTED = DistributedContext()
_current: contextvars.ContextVar[DistributedContext] = contextvars.ContextVar("nva_dd_context", default=NOT_DISTRIBUTED)


def current_dd_context() -> DistributedContext:
    return _current.get()


@contextlib.contextmanager
def activate_dd_context(ctx: DistributedContext) -> Iterator[DistributedContext]:
    token = _current.set(ctx)
    try:
        yield ctx
    finally:
        _current.reset(token)


@dataclass
class ShardRouting:
    """Tables that translate between global atom ids and ``(owner rank, index on the owner)``."""

    owner: torch.Tensor          # [N] owner rank of each global id
    local_index: torch.Tensor    # [N] position of the atom on its owner (owners keep ascending global id order)
    counts: torch.Tensor         # [world] atoms per rank
    offsets: torch.Tensor        # [world + 1]

    @classmethod
    def from_assignment(cls, owner: torch.Tensor, world_size: int) -> "ShardRouting":
        owner = owner.long()
        counts = torch.bincount(owner, minlength=world_size)
        offsets = torch.zeros(world_size + 1, dtype=torch.long, device=owner.device)
        offsets[1:] = torch.cumsum(counts, 0)
        order = torch.argsort(owner, stable=True)  # global ids grouped by owner, ascending inside each group
        local = torch.empty_like(owner)
        local[order] = torch.arange(owner.numel(), device=owner.device) - offsets[owner[order]]
        return cls(owner, local, counts, offsets)

    def global_ids_of(self, rank: int) -> torch.Tensor:
        return torch.nonzero(self.owner == rank, as_tuple=False).flatten()

    def to_flat(self, global_ids: torch.Tensor) -> torch.Tensor:
        """Index into the rank-ordered concatenation of all ranks' owned rows."""
        g = global_ids.long()
        return self.offsets[self.owner[g]] + self.local_index[g]


def reshard_by_destination(rows: torch.Tensor, destination: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Send each row to the rank named in ``destination``; returns the rows received (ordered by source rank)."""
    from nvalchemi_toolkit_b200.distributed.halo import migrate_rows

    return migrate_rows({"rows": rows}, destination.long(), group)["rows"]
