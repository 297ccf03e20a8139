# SPDX-License-Identifier: Apache-2.0
"""Fixed-shape halo exchange: the same ghost refresh and ghost fold as :class:`HaloExchange`, with every tensor shape
pinned by two capacities, so a step has the same launch sequence whatever the current ghost count.

Reference: ``halo_forward_static`` / ``halo_scatter_correct_static`` with packed routing tensors
(``nvalchemi/distributed/_core/particle_halo.py:1190-1327``), which exist there so that a ``torch.compile``-d step is not
re-traced when the ghost lists change.  Nothing is traced here; the fixed shapes serve CUDA-graph capture of a step
(``all_to_all_single`` with uniform splits is capturable, a variable-split exchange is not) and allocation-free steady
state: between list rebuilds no tensor of a different size is ever created.

Layout.  A padded node tensor has ``n_padded`` rows: ``[owned rows | ghost rows | unused rows]``.  Every rank sends at
most ``max_send`` rows to every other rank (uniform splits; unused slots carry row 0 of the sender and are masked out at
the receiver).  :class:`StaticHaloRouting` packs the plan of a built :class:`HaloExchange` into four device tensors

* ``send_index [world * max_send]``: owned row that fills each send slot,
* ``recv_dest  [world * max_send]``: padded row each received slot lands in (ghost rows are stored in arrival order),
* ``recv_real  [world * max_send]``: which received slots are real,
* ``n_owned    []``: first ghost row,

which can be refreshed IN PLACE after a list rebuild (same shapes), so a captured graph that reads them stays valid.
The capacities are agreed over the ranks with ``graph_padder.resolve_cap`` (every rank must use the same ``max_send``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.distributed.halo import HaloExchange, _world


def halo_exchange_fixed(rows: torch.Tensor, world: int, group: Any = None) -> torch.Tensor:
    """Uniform-split all-to-all of ``[world * k, ...]`` rows: block ``r`` goes to rank ``r``."""
    if world == 1 or not dist.is_initialized():
        return rows.clone()
    out = torch.empty_like(rows)
    dist.all_to_all_single(out, rows.contiguous(), group=group)
    return out


@dataclass
class StaticHaloRouting:
    send_index: torch.Tensor
    recv_dest: torch.Tensor
    recv_real: torch.Tensor
    send_real: torch.Tensor
    n_owned: torch.Tensor
    world: int
    max_send: int
    n_padded: int
    group: Any = None

    @classmethod
    def allocate(cls, world: int, max_send: int, n_padded: int, device: torch.device | str, group: Any = None) -> "StaticHaloRouting":
        k = world * max_send
        z = lambda dt: torch.zeros(k, dtype=dt, device=device)  # noqa: E731
        return cls(z(torch.int64), z(torch.int64), z(torch.bool), z(torch.bool), torch.zeros((), dtype=torch.int64, device=device),
                   world, max_send, n_padded, group)

    @classmethod
    def from_halo(cls, halo: HaloExchange, n_owned: int, max_send: int, n_padded: int) -> "StaticHaloRouting":
        rank, world = _world(halo.group)
        out = cls.allocate(world, max_send, n_padded, halo.send_index.device, halo.group)
        out.update_(halo, n_owned)
        return out

    def update_(self, halo: HaloExchange, n_owned: int) -> "StaticHaloRouting":
        """Re-pack the plan of a (re)built exchange into the existing tensors.  Raises when a capacity is exceeded: the
        caller then grows the capacities on all ranks together and re-captures."""
        if max(halo.send_splits, default=0) > self.max_send or max(halo.recv_splits, default=0) > self.max_send:
            raise OverflowError(f"halo plan sends up to {max(max(halo.send_splits, default=0), max(halo.recv_splits, default=0))} "
                                f"rows to one rank, capacity max_send = {self.max_send}")
        if n_owned + halo.n_ghost > self.n_padded:
            raise OverflowError(f"{n_owned} owned + {halo.n_ghost} ghost rows exceed n_padded = {self.n_padded}")
        dev = self.send_index.device
        slot = torch.arange(self.max_send, device=dev)
        send_cnt = torch.tensor(halo.send_splits, device=dev)
        recv_cnt = torch.tensor(halo.recv_splits, device=dev)
        send_off = torch.cumsum(send_cnt, 0) - send_cnt
        recv_off = torch.cumsum(recv_cnt, 0) - recv_cnt
        s_real = slot[None, :] < send_cnt[:, None]                       # [world, max_send]
        r_real = slot[None, :] < recv_cnt[:, None]
        s_src = (send_off[:, None] + slot[None, :]).clamp_max(max(int(halo.send_index.numel()) - 1, 0))
        sidx = halo.send_index[s_src.reshape(-1)] if halo.send_index.numel() else torch.zeros(s_src.numel(), dtype=torch.int64, device=dev)
        self.send_index.copy_(torch.where(s_real.reshape(-1), sidx, torch.zeros_like(sidx)))
        self.send_real.copy_(s_real.reshape(-1))
        dest = n_owned + recv_off[:, None] + slot[None, :]
        self.recv_dest.copy_(torch.where(r_real, dest, torch.zeros_like(dest)).reshape(-1))
        self.recv_real.copy_(r_real.reshape(-1))
        self.n_owned.fill_(n_owned)
        return self


def _mask(flags: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    return flags.reshape((-1,) + (1,) * (like.dim() - 1))


def _refresh(padded: torch.Tensor, r: StaticHaloRouting) -> torch.Tensor:
    """Owned rows pass through; ghost rows are overwritten with their owners' current rows; unused rows become zero."""
    recv = halo_exchange_fixed(padded.index_select(0, r.send_index), r.world, r.group)
    recv = recv * _mask(r.recv_real, recv).to(recv.dtype)
    ghosts = torch.zeros_like(padded).index_add_(0, r.recv_dest, recv)   # masked slots add zero to row 0
    rows = torch.arange(padded.shape[0], device=padded.device)
    return torch.where(_mask(rows >= r.n_owned, padded), ghosts, padded)


def _fold(padded: torch.Tensor, r: StaticHaloRouting) -> torch.Tensor:
    """Ghost-row partial sums travel back and are added to the owners' rows; ghost rows of the result are zero."""
    rows = torch.arange(padded.shape[0], device=padded.device)
    ghost = _mask(rows >= r.n_owned, padded)
    back = padded.index_select(0, r.recv_dest) * _mask(r.recv_real, padded).to(padded.dtype)
    back = halo_exchange_fixed(back, r.world, r.group)
    back = back * _mask(r.send_real, back).to(back.dtype)
    own = torch.where(ghost, torch.zeros_like(padded), padded)
    return own.index_add(0, r.send_index, back)


class _ForwardStatic(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, padded: torch.Tensor, routing: StaticHaloRouting) -> torch.Tensor:
        ctx.routing = routing
        return _refresh(padded, routing)

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        return _fold(grad.contiguous(), ctx.routing), None  # gradients on ghost copies belong to the owners


class _ScatterCorrectStatic(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, padded: torch.Tensor, routing: StaticHaloRouting) -> torch.Tensor:
        ctx.routing = routing
        return _refresh(_fold(padded, routing), routing)

    @staticmethod
    def backward(ctx: Any, grad: torch.Tensor) -> tuple[torch.Tensor, None]:
        # adjoint of refresh o fold: fold^T o refresh^T, with refresh^T = fold and fold^T = refresh on owned-only input
        return _refresh(_fold(grad.contiguous(), ctx.routing), ctx.routing), None


def halo_forward_static(padded: torch.Tensor, routing: StaticHaloRouting) -> torch.Tensor:
    """``[owned | stale ghosts | unused] -> [owned | fresh ghosts | 0]``, differentiable, fixed shapes."""
    return _ForwardStatic.apply(padded, routing)


def halo_scatter_correct_static(padded: torch.Tensor, routing: StaticHaloRouting) -> torch.Tensor:
    """After a scatter that left partial sums on ghost rows: fold them into the owners, then refresh every ghost row with
    its owner's completed value, so that owned AND ghost rows hold the full sums.  Differentiable, fixed shapes."""
    return _ScatterCorrectStatic.apply(padded, routing)


class StaticHalo:
    """Capacity management around :class:`StaticHaloRouting`: capacities come from ``graph_padder.resolve_cap`` (grow-only,
    bucketed, agreed over the ranks of the exchange's group), the routing tensors are re-packed in place after every
    rebuild of the exchange, and only a capacity overflow allocates new tensors (``generation`` then changes: the signal
    for a consumer that captured a CUDA graph over the old ones to capture again)."""

    def __init__(self, halo: HaloExchange) -> None:
        self.halo = halo
        self.caps: dict[str, int] = {}
        self.routing: StaticHaloRouting | None = None
        self.generation = 0
        self._packed_build = -1

    def sync(self, n_owned: int) -> StaticHaloRouting:
        """Routing for the exchange's CURRENT plan (call after ``halo.build``; cheap when nothing changed)."""
        from nvalchemi_toolkit_b200.distributed.graph_padder import cap_agreement_group, resolve_cap

        halo = self.halo
        if self.routing is not None and self._packed_build == halo.num_builds and int(self.routing.n_owned) == n_owned:
            return self.routing
        dev = halo.send_index.device
        per_peer = max(max(halo.send_splits, default=0), max(halo.recv_splits, default=0))
        with cap_agreement_group(halo.group, dev):
            max_send = resolve_cap(self.caps, "max_send", per_peer)
            n_padded = resolve_cap(self.caps, "n_padded", n_owned + halo.n_ghost)
        r = self.routing
        if r is None or r.max_send != max_send or r.n_padded != n_padded:
            _, world = _world(halo.group)
            self.routing = StaticHaloRouting.allocate(world, max_send, n_padded, dev, halo.group)
            self.generation += 1
        self.routing.update_(halo, n_owned)
        self._packed_build = halo.num_builds
        return self.routing

    def pad(self, owned: torch.Tensor) -> torch.Tensor:
        """``[n_owned, ...] -> [n_padded, ...]`` with zero ghost and unused rows (input of :func:`halo_forward_static`)."""
        r = self.routing
        out = owned.new_zeros((r.n_padded,) + tuple(owned.shape[1:]))
        out[: owned.shape[0]] = owned
        return out

    def refresh(self, owned: torch.Tensor) -> torch.Tensor:
        """Owned rows -> padded tensor with current ghost rows (differentiable)."""
        return halo_forward_static(self.pad(owned), self.routing)
