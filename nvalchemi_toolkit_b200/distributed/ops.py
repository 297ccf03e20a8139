# SPDX-License-Identifier: Apache-2.0
"""Differentiable halo primitives and the explicit ``ShardTensor`` container.

Reference: ``nvalchemi/distributed/ops.py:110-720`` and ``_core/shard_tensor.py``.  The reference subclasses
``torch.Tensor`` and intercepts ``index_select`` / ``scatter_add`` through ``__torch_dispatch__``; here the same data
movement is exposed as explicit autograd functions, which is what a hand-written distributed forward (or a training
step across sub-domains) calls:

* :func:`halo_forward`: ghost rows from owners; its backward adds ghost-row gradients back into the owners.
* :func:`halo_scatter_correct`: after a scatter-add over local edges, partial sums that landed on ghost rows are
  added into their owners; its backward forwards owner gradients to the ghosts.
"""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.distributed.halo import HaloExchange


class _HaloForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, owned: torch.Tensor, halo: HaloExchange) -> torch.Tensor:
        ctx.halo = halo
        return torch.cat([owned, halo.forward(owned)])

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        n = grad.shape[0] - ctx.halo.n_ghost
        own = grad[:n].clone()
        ctx.halo.reverse_add(grad[n:].contiguous(), own)
        return own, None


class _HaloScatterCorrect(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, padded: torch.Tensor, halo: HaloExchange) -> torch.Tensor:
        ctx.halo = halo
        n = padded.shape[0] - halo.n_ghost
        own = padded[:n].clone()
        halo.reverse_add(padded[n:].contiguous(), own)
        return own

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        return torch.cat([grad, ctx.halo.forward(grad.contiguous())]), None


class _GatherReplicate(torch.autograd.Function):
    """All ranks' rows concatenated in rank order; the adjoint sums every rank's gradient of this rank's rows."""

    @staticmethod
    def forward(ctx: Any, owned: torch.Tensor, group: Any) -> torch.Tensor:
        from nvalchemi_toolkit_b200.distributed.halo import _world, all_gather_rows

        rows, counts = all_gather_rows(owned.contiguous(), group)
        rank, _ = _world(group)
        ctx.group, ctx.start, ctx.n = group, int(sum(counts[:rank])), owned.shape[0]
        return rows

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        import torch.distributed as dist

        g = grad.contiguous().clone()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g[ctx.start: ctx.start + ctx.n], None


def gather_replicate(owned: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Differentiable all-gather of row blocks (rank order)."""
    return _GatherReplicate.apply(owned, group)


def per_system_reduce(values: torch.Tensor, index: torch.Tensor, n_systems: int, group: Any = None) -> torch.Tensor:
    """Sum of OWNED per-atom values per system, all-reduced over the ranks (reference
    ``nvalchemi/distributed/_core/per_system.py:68-213``); differentiable: every rank's gradient of the replicated
    result is summed before it flows back to the local rows."""
    local = values.new_zeros((n_systems,) + tuple(values.shape[1:])).index_add(0, index.long(), values)
    return _AllReduceSum.apply(local, group)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, group: Any) -> torch.Tensor:
        import torch.distributed as dist

        ctx.group = group
        y = x.contiguous().clone()
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        import torch.distributed as dist

        g = grad.contiguous().clone()
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


def distributed_all_reduce(x: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Differentiable sum over the ranks of the group."""
    return _AllReduceSum.apply(x, group)


def halo_forward(owned: torch.Tensor, halo: HaloExchange) -> torch.Tensor:
    return _HaloForward.apply(owned, halo)


def halo_scatter_correct(padded: torch.Tensor, halo: HaloExchange) -> torch.Tensor:
    return _HaloScatterCorrect.apply(padded, halo)


class ShardTensor:
    """A per-atom tensor split by sub-domain: ``local`` holds the owned rows; :meth:`padded` appends current ghost
    rows, :meth:`fold` returns ghost-row partial sums to the owners, :meth:`full_tensor` gathers all ranks' rows in
    global-id order.  An explicit container, not a ``torch.Tensor`` subclass."""

    def __init__(self, local: torch.Tensor, sharded: Any) -> None:
        self.local, self.sharded = local, sharded

    @property
    def n_owned(self) -> int:
        return self.local.shape[0]

    def to_local(self) -> torch.Tensor:
        return self.local

    def padded(self) -> torch.Tensor:
        return halo_forward(self.local, self.sharded.halo)

    @staticmethod
    def fold(padded: torch.Tensor, sharded: Any) -> "ShardTensor":
        return ShardTensor(halo_scatter_correct(padded, sharded.halo), sharded)

    def full_tensor(self) -> torch.Tensor:
        from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows

        rows, _ = all_gather_rows(self.local.detach().contiguous(), self.sharded.group)
        ids, _ = all_gather_rows(self.sharded.global_ids, self.sharded.group)
        return rows[torch.argsort(ids)]


# The "mechanism" namespace (reference ``nvalchemi/distributed/ops.py``): everything a hand-written distributed forward
# needs, importable from one place.
from nvalchemi_toolkit_b200.distributed._runtime import mesh_group  # noqa: E402
from nvalchemi_toolkit_b200.distributed.collectives import (distributed_index_select, distributed_scatter_add,  # noqa: E402
                                                            gather_to_replicate)
from nvalchemi_toolkit_b200.distributed.context import (NOT_DISTRIBUTED, DistributedContext, ShardRouting,  # noqa: E402
                                                        activate_dd_context, current_dd_context)
from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows, all_to_all_rows, neighbor_exchange_rows  # noqa: E402
from nvalchemi_toolkit_b200.distributed.storage_policy import (GraphParallelPolicy, HaloStoragePolicy, PlainShard,  # noqa: E402
                                                               RefreshOnlyHaloPolicy, StoragePolicy)

__all__ = ["halo_forward", "halo_scatter_correct", "gather_replicate", "per_system_reduce", "distributed_all_reduce",
           "ShardTensor", "mesh_group", "distributed_index_select", "distributed_scatter_add", "gather_to_replicate",
           "DistributedContext", "NOT_DISTRIBUTED", "ShardRouting", "activate_dd_context", "current_dd_context",
           "all_gather_rows", "all_to_all_rows", "neighbor_exchange_rows", "StoragePolicy", "PlainShard",
           "HaloStoragePolicy", "RefreshOnlyHaloPolicy", "GraphParallelPolicy"]
