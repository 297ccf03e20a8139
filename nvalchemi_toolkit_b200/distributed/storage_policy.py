# SPDX-License-Identifier: Apache-2.0
"""Storage policies: how the rows a rank holds of a per-atom tensor relate to the global tensor, and what has to
happen when a model gathers from it or scatters into it.

Reference: ``nvalchemi/distributed/_core/storage_policy.py:140-596`` (``StoragePolicy`` protocol, ``PlainShard``,
``HaloStoragePolicy(scatter_mode, gather_mode)``, ``RefreshOnlyHaloPolicy``, ``GraphParallelPolicy``, the
``policy_to_dict`` / ``policy_from_dict`` registry).  A policy has two hooks used once per message-passing layer by
:class:`~nvalchemi_toolkit_b200.distributed.dispatch.HaloDispatchMode`:

* ``replicate(x, ctx)``: make the rows other atoms will *read* current (ghost refresh from the owners, or an
  all-gather of every rank's rows);
* ``fold(out, ctx)``: after a scatter over local edges, return partial sums that landed on rows this rank does not own
  to their owners.

Both are differentiable (their adjoints communicate in the backward pass).  ``ctx`` is any object with ``halo``
(:class:`~nvalchemi_toolkit_b200.distributed.halo.HaloExchange`), ``n_owned`` and ``group``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Protocol, runtime_checkable

import torch

__all__ = ["StoragePolicy", "PlainShard", "HaloStoragePolicy", "RefreshOnlyHaloPolicy", "GraphParallelPolicy",
           "row_offsets", "policy_to_dict", "policy_from_dict", "register_policy_kind"]


def row_offsets(sizes: list[int]) -> list[int]:
    """Prefix sums of per-rank row counts (length ``world + 1``)."""
    out = [0]
    for s in sizes:
        out.append(out[-1] + int(s))
    return out


@runtime_checkable
class StoragePolicy(Protocol):
    kind: str

    @property
    def partition_mode(self) -> str: ...

    def to_local(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor: ...

    def full_tensor(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor: ...

    def replicate(self, x: torch.Tensor, ctx: Any) -> torch.Tensor: ...

    def fold(self, out: torch.Tensor, ctx: Any) -> torch.Tensor: ...

    def to_dict(self) -> dict: ...


def _gather_in_id_order(owned: torch.Tensor, ctx: Any) -> torch.Tensor:
    from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows

    rows, _ = all_gather_rows(owned.detach().contiguous(), ctx.group)
    ids = getattr(ctx, "global_ids", None)
    if ids is None:
        return rows
    all_ids, _ = all_gather_rows(ids.contiguous(), ctx.group)
    return rows[torch.argsort(all_ids)]


@dataclass(frozen=True)
class PlainShard:
    """Each rank stores exactly its owned rows; reads and scatters stay local."""

    kind: str = "plain_shard"

    @property
    def partition_mode(self) -> str:
        return "shard"

    def to_local(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor:
        return stored

    def full_tensor(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor:
        return _gather_in_id_order(stored, ctx)

    def replicate(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        return x

    def fold(self, out: torch.Tensor, ctx: Any) -> torch.Tensor:
        return out

    def to_dict(self) -> dict:
        return {"kind": self.kind}


@dataclass(frozen=True)
class HaloStoragePolicy:
    """Owned rows followed by borrowed (ghost) rows.

    ``gather_mode``: ``"halo_read"`` refreshes the ghost rows from their owners before a gather, ``"local"`` reads what
    is there.  ``scatter_mode``: ``"halo_correction"`` adds the partial sums accumulated on ghost rows into the owners'
    rows after a scatter (needed when edges whose receiver is a ghost are kept), ``"local"`` leaves them.

    Folding is only right for an edge-partitioned graph (every edge evaluated on exactly one rank): with this policy
    ``DistributedModel`` keeps, on each rank, the edges whose sender it owns (``_keep_owned_senders``).
    """

    scatter_mode: str = "halo_correction"
    gather_mode: str = "halo_read"
    kind: str = "halo"

    def __post_init__(self) -> None:
        if self.scatter_mode not in ("halo_correction", "local") or self.gather_mode not in ("halo_read", "local"):
            raise ValueError(f"unknown modes ({self.scatter_mode!r}, {self.gather_mode!r})")

    @property
    def partition_mode(self) -> str:
        return "halo"

    def to_local(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor:
        return stored[: ctx.n_owned]

    def full_tensor(self, stored: torch.Tensor, ctx: Any) -> torch.Tensor:
        return _gather_in_id_order(stored[: ctx.n_owned], ctx)

    def replicate(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        if self.gather_mode == "local":
            return x
        from nvalchemi_toolkit_b200.distributed.ops import halo_forward

        return halo_forward(x[: ctx.n_owned], ctx.halo)

    def fold(self, out: torch.Tensor, ctx: Any) -> torch.Tensor:
        if self.scatter_mode == "local":
            return out
        from nvalchemi_toolkit_b200.distributed.ops import halo_scatter_correct

        own = halo_scatter_correct(out, ctx.halo)
        return torch.cat([own, out.new_zeros((out.shape[0] - own.shape[0],) + tuple(out.shape[1:]))])

    def to_dict(self) -> dict:
        return {"kind": self.kind, "scatter_mode": self.scatter_mode, "gather_mode": self.gather_mode}


@dataclass(frozen=True)
class RefreshOnlyHaloPolicy(HaloStoragePolicy):
    """Halo storage for owned-complete aggregation: every edge that ends on an owned atom is present locally (the ghost
    layer is one cutoff deep), so a scatter leaves the owned rows complete and nothing has to be folded; only the
    ghost rows must be refreshed before the next gather."""

    scatter_mode: str = "local"
    gather_mode: str = "halo_read"
    kind: str = "halo_refresh_only"


@dataclass(frozen=True)
class GraphParallelPolicy(PlainShard):
    """Balanced index blocks with replicated geometry: reads see every rank's rows (all-gather whose adjoint is a
    reduce-scatter), scatters produce owned rows only."""

    kind: str = "graph_parallel"

    @property
    def partition_mode(self) -> str:
        return "graph_partition"

    def replicate(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows
        from nvalchemi_toolkit_b200.distributed.ops import gather_replicate

        rows = gather_replicate(x, ctx.group)
        ids = getattr(ctx, "global_ids", None)
        if ids is None:
            return rows
        all_ids, _ = all_gather_rows(ids.contiguous(), ctx.group)
        return rows[torch.argsort(all_ids)]


_KINDS: dict[str, Callable[[dict], Any]] = {
    "plain_shard": lambda d: PlainShard(),
    "halo": lambda d: HaloStoragePolicy(d.get("scatter_mode", "halo_correction"), d.get("gather_mode", "halo_read")),
    "halo_refresh_only": lambda d: RefreshOnlyHaloPolicy(d.get("scatter_mode", "local"), d.get("gather_mode", "halo_read")),
    "graph_parallel": lambda d: GraphParallelPolicy(),
}


def register_policy_kind(kind: str, from_dict: Callable[[dict], Any]) -> None:
    _KINDS[kind] = from_dict


def policy_to_dict(policy: Any) -> dict:
    return policy.to_dict()


def policy_from_dict(d: dict) -> Any:
    try:
        return _KINDS[d["kind"]](d)
    except KeyError as e:
        raise ValueError(f"unknown storage policy kind {d.get('kind')!r}; known: {sorted(_KINDS)}") from e
