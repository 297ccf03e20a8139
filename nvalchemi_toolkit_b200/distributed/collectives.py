# SPDX-License-Identifier: Apache-2.0
"""Collectives addressed by GLOBAL atom id (reference ``nvalchemi/distributed/_core/gather_primitives.py``,
``_core/collectives.py``): fetch rows owned by other ranks, add contributions into rows owned by other ranks, replicate
a sharded tensor.  Built on the variable-size all-to-all of :mod:`halo`; each call is two message rounds (indices,
then rows)."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.distributed.context import ShardRouting
from nvalchemi_toolkit_b200.distributed.halo import _world, all_gather_rows, all_to_all_rows, exchange_counts


def _by_owner(global_ids: torch.Tensor, routing: ShardRouting, world: int) -> tuple[torch.Tensor, list[int]]:
    owner = routing.owner.to(global_ids.device)[global_ids.long()]
    order = torch.argsort(owner, stable=True)
    return order, torch.bincount(owner, minlength=world).tolist()


def distributed_index_select(local_rows: torch.Tensor, global_ids: torch.Tensor, routing: ShardRouting, group: Any = None
                             ) -> torch.Tensor:
    """Rows of a sharded per-atom tensor for arbitrary global ids (``local_rows`` are this rank's owned rows in ascending
    global-id order)."""
    rank, world = _world(group)
    local_index = routing.local_index.to(global_ids.device)
    if world == 1:
        return local_rows[local_index[global_ids.long()]]
    order, counts = _by_owner(global_ids, routing, world)
    recv_counts = exchange_counts(counts, global_ids.device, group)
    wanted = all_to_all_rows(local_index[global_ids.long()][order], counts, recv_counts, group)  # indices peers ask of me
    rows = all_to_all_rows(local_rows[wanted], recv_counts, counts, group)
    out = torch.empty_like(rows)
    out[order] = rows
    return out


def distributed_scatter_add(local_rows: torch.Tensor, global_ids: torch.Tensor, values: torch.Tensor, routing: ShardRouting,
                            group: Any = None) -> torch.Tensor:
    """``local_rows[owner-local index of id] += value`` for contributions addressed to any rank's atoms (in place)."""
    rank, world = _world(group)
    local_index = routing.local_index.to(global_ids.device)
    if world == 1:
        return local_rows.index_add_(0, local_index[global_ids.long()], values.to(local_rows.dtype))
    order, counts = _by_owner(global_ids, routing, world)
    recv_counts = exchange_counts(counts, global_ids.device, group)
    idx = all_to_all_rows(local_index[global_ids.long()][order], counts, recv_counts, group)
    vals = all_to_all_rows(values[order].contiguous(), counts, recv_counts, group)
    return local_rows.index_add_(0, idx, vals.to(local_rows.dtype))


def gather_to_replicate(local_rows: torch.Tensor, global_ids: torch.Tensor, group: Any = None) -> torch.Tensor:
    """The full tensor in global-id order on every rank."""
    rows, _ = all_gather_rows(local_rows.contiguous(), group)
    ids, _ = all_gather_rows(global_ids.contiguous(), group)
    return rows[torch.argsort(ids)]
