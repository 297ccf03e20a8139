# SPDX-License-Identifier: Apache-2.0
"""Helpers a model author uses to stay correct with and without domain decomposition.

Reference: ``nvalchemi/distributed/helpers.py:40-510`` (``to_local``, ``scatter_to_owners``, ``system_sum``,
``refresh_neighbors``, ``gather_replicated``): each is an identity (or a plain local reduction) when no process group is
active, so the same model code runs single-process.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.distributed.halo import _world, all_gather_rows


def to_local(t: Any) -> torch.Tensor:
    """The rank-local tensor behind ``t`` (``ShardTensor`` → its local rows; plain tensors unchanged)."""
    return t.local if hasattr(t, "local") and hasattr(t, "n_owned") else t


def system_sum(values: torch.Tensor, batch_idx: torch.Tensor, num_systems: int, weights: torch.Tensor | None = None,
               group: Any = None, distributed: bool = False) -> torch.Tensor:
    """Per-system sum of per-atom ``values`` (optionally weighted: 0 on ghost rows), all-reduced when ``distributed``."""
    v = values if weights is None else values * weights.reshape((-1,) + (1,) * (values.dim() - 1)).to(values.dtype)
    out = v.new_zeros((num_systems,) + tuple(v.shape[1:])).index_add_(0, batch_idx.long(), v)
    if distributed and _world(group)[1] > 1:
        dist.all_reduce(out, group=group)
    return out


def scatter_to_owners(ghost_rows: torch.Tensor, owned_rows: torch.Tensor, sharded: Any = None) -> torch.Tensor:
    """Add contributions computed on ghost rows into their owners' rows (identity without a sharded batch)."""
    if sharded is None:
        return owned_rows
    return sharded.halo.reverse_add(ghost_rows, owned_rows)


def refresh_ghosts(owned_rows: torch.Tensor, sharded: Any = None) -> torch.Tensor:
    """``[owned; ghost]`` rows of a per-atom tensor, ghosts fetched from their owners (per-layer feature refresh)."""
    if sharded is None:
        return owned_rows
    return torch.cat([owned_rows, sharded.halo.forward(owned_rows)])


def refresh_neighbors(batch: Any, hook: Any) -> None:
    """Run a neighbour-list hook outside a dynamics loop."""
    from types import SimpleNamespace

    hook(SimpleNamespace(batch=batch), None)


def gather_replicated(rows: torch.Tensor, group: Any = None) -> torch.Tensor:
    """Every rank's rows concatenated in rank order (graph-partition strategy: features replicated per layer)."""
    return all_gather_rows(rows, group)[0]


def total_charge_correction(charges: torch.Tensor, total_charge: torch.Tensor, batch_idx: torch.Tensor,
                            weights: torch.Tensor | None = None, group: Any = None, distributed: bool = False
                            ) -> torch.Tensor:
    """Shift per-atom charges uniformly so that each system sums to ``total_charge`` (sums and counts are global)."""
    nb = total_charge.reshape(-1).shape[0]
    w = torch.ones_like(charges) if weights is None else weights.to(charges.dtype)
    q = system_sum(charges, batch_idx, nb, w, group, distributed)
    n = system_sum(torch.ones_like(charges), batch_idx, nb, w, group, distributed)
    delta = (total_charge.reshape(-1).to(charges.dtype) - q) / n.clamp_min(1)
    return charges + delta[batch_idx.long()]


def localize(data: dict[str, Any]) -> dict[str, Any]:
    """:func:`to_local` over every value of a model-input dictionary (a shallow copy; non-tensor entries pass through)."""
    return {k: to_local(v) for k, v in data.items()}


def autograd_target(t: Any) -> torch.Tensor:
    """The tensor to hand to ``torch.autograd.grad(inputs=...)`` for a quantity the framework may have wrapped.  Node
    tensors stay plain tensors in this package (the distributed forward is a mode, not a tensor subclass), so this is
    the identity except for a :class:`ShardTensor` container, whose padded local tensor is the leaf in the graph."""
    if hasattr(t, "autograd_target") and callable(t.autograd_target):
        return t.autograd_target()
    return t.local if hasattr(t, "local") and hasattr(t, "n_owned") else t


def distributed_method(body: Any) -> Any:
    """Decorator for the replacement function of a ``MethodAdapter`` / ``PythonAdapter`` that only differs under domain
    decomposition (reference ``distributed/helpers.py:103-143``).  ``body(original, mode, *args, **kwargs)`` runs inside a
    distributed forward, with the active dispatch mode in hand; everywhere else the original is called unchanged, so the
    guard does not have to be repeated in every adapter::

        @distributed_method
        def mol_sum(original, mode, x, mol_idx):
            return per_system_reduce(x * mode.owned_mask(x), mol_idx, n_systems, mode.group)
        PythonAdapter("aimnet.nbops", "mol_sum", mol_sum(aimnet.nbops.mol_sum))   # decorated(original) -> replacement
    """
    import functools

    from nvalchemi_toolkit_b200.distributed.dispatch import current_dispatch

    @functools.wraps(body)
    def bound(original: Any) -> Any:
        @functools.wraps(original)
        def replacement(*args: Any, **kwargs: Any) -> Any:
            mode = current_dispatch()
            if mode is None:
                return original(*args, **kwargs)
            return body(original, mode, *args, **kwargs)

        return replacement

    bound.__distributed_method__ = True  # type: ignore[attr-defined]
    return bound


def neighbor_refresh_adapters(modules: Any, *, output: int = 0) -> tuple:
    """One ``ModuleForwardAdapter`` per concrete class among ``modules`` (e.g. ``model.interactions``) whose ``forward``
    scatters messages into a per-node output the dispatch mode cannot see (a fused or scripted block): forward output
    ``output`` is folded per the storage policy and marked stale, so the next gather refreshes its ghost rows
    (reference ``distributed/helpers.py:146-200``).  Outside a distributed forward the adapters do nothing."""
    from nvalchemi_toolkit_b200.distributed.dispatch import ModuleForwardAdapter

    mods = list(modules.values()) if isinstance(modules, dict) else (list(modules) if isinstance(modules, (list, tuple, torch.nn.ModuleList)) else [modules])
    classes: list[type] = []
    for m in mods:
        cls = next((c for c in type(m).__mro__ if "forward" in c.__dict__), None)
        if cls is not None and cls not in classes:
            classes.append(cls)
    return tuple(ModuleForwardAdapter(c, node_outputs=(output,)) for c in classes)
