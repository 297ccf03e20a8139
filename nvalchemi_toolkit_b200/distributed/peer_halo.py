# SPDX-License-Identifier: Apache-2.0
"""Peer-memory halo engine: the native MACE evaluated on one rank's owned + ghost rows, with every ghost exchange done
by this package's NVLink kernels over symmetric (peer-mapped) buffers.

It is the fast backend of :class:`DistributedModel` for a :class:`ShardedBatch` decomposed by
:class:`SpatialPartitioner` (any 3-D rank grid).  What the reference does with ``HaloStrategy`` + ShardTensor dispatch
(``nvalchemi/distributed/strategy.py:680-911``, ``distributed/_core/particle_halo.py:279-368,557-638``,
``distributed/output_consolidation.py:316-340``) becomes:

* **plan** (rebuilt with the ghost lists, i.e. when the skin is exhausted): the send/receive plan of
  :class:`HaloExchange` is turned into *pull tables*: for every ghost row its owner rank, its row on the owner and
  its integer lattice shift.  Only the ranks that share ghosts exchange anything (row indices, 4 bytes per ghost);
* **per step**: owned positions are written into the symmetric position buffer, a flag barrier orders them, the ghost
  positions are pulled from the owners (P2P loads + shift), the neighbour list is built over owned + ghost rows with
  rows for owned atoms only, and the network runs on the owned atoms.  Before each interaction the ghost rows of the
  sender features are pulled from their owners (16-byte loads, one warp per row, only rows some local edge uses); in the
  adjoint the gradients accumulated on ghost rows are returned with vector reductions.  Each edge is evaluated once (at
  the owner of its receiver) and energies are sums over owned atoms, so no ``/ world_size`` bookkeeping exists;
* **sums**: the energy (and the virial when stress is requested) is all-reduced in float64.

No TMA is involved in any peer access; the buffers are touched with plain loads, stores and reductions only.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.distributed.graph_padder import cap_agreement_group, resolve_cap
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


from nvalchemi_toolkit_b200.distributed.failure import PeerFailure  # noqa: E402  (re-exported)


def peer_memory_available(wrapper: Any, device: torch.device, group: Any) -> bool:
    """Can this (model, device, process group) use the peer-memory engine?"""
    from nvalchemi_toolkit_b200.models.mace.wrapper import MACEWrapper
    from nvalchemi_toolkit_b200.ops import _native

    if not (dist.is_available() and dist.is_initialized()) or device.type != "cuda":
        return False
    if dist.get_world_size(group) < 2 or dist.get_backend(group) != "nccl":
        return False
    if not isinstance(wrapper, MACEWrapper) or wrapper.model.backend == "torch" or wrapper.training:
        return False
    if next(wrapper.model.parameters()).dtype != torch.float32:
        return False
    return _native.available()


def build_pull_tables(sharded: Any) -> dict[str, torch.Tensor]:
    """Pull tables of a sharded batch's ghost plan (pure ``torch`` + the plan's own exchanges; any backend).

    ``home_rank [G] int32`` / ``home_row [G] int32``: owner rank of every ghost row and its row among the owner's atoms;
    ``ghost_image [G, 3]``: lattice image to add (times the cell) to the owner's row *as the owner stores it*, i.e. in
    the owner's frame ``positions + wrap_image @ cell``; ``wrap_image [N_owned, 3]``: this rank's own frame;
    ``send_row / send_peer / send_peer_row / send_used_index [S]``: for every row this rank sends, its own row, the rank
    that holds the copy, the copy's row in that rank's local numbering and its index among that rank's ghosts."""
    halo = sharded.halo
    n = sharded.n_owned
    dev = sharded.owned.positions.device
    image = halo.send_shift - halo.wrap_shift[halo.send_index]  # image relative to the owner's own frame
    ng = halo.n_ghost
    ghost_ids = torch.arange(ng, dtype=torch.int32, device=dev)
    world = max(1, len(halo.send_splits))
    return {
        # reverse path (owner pulls): for every row this rank sends, the rank holding the copy and the copy's row there
        "send_row": halo.send_index.to(torch.int32).contiguous(),
        "send_peer": torch.repeat_interleave(torch.arange(world, dtype=torch.int32, device=dev),
                                             torch.tensor(halo.send_splits, device=dev)).contiguous(),
        "send_used_index": halo.reverse_packed(ghost_ids).contiguous(),
        "send_peer_row": halo.reverse_packed(ghost_ids + n).contiguous(),
        "home_rank": halo.ghost_owner_rank.to(torch.int32).contiguous(),
        "home_row": halo.forward(torch.arange(n, dtype=torch.int32, device=dev)).contiguous(),
        "ghost_image": halo.forward_packed(image.to(torch.float32).contiguous()).contiguous(),
        "wrap_image": halo.wrap_shift.to(torch.float32).contiguous(),
    }


class PeerHaloEngine:
    """Symmetric arena, pull tables and the per-step evaluation for one ``ShardedBatch``."""

    #: rows are pulled / returned in bulk once per layer (the convolution kernels then work on local memory)
    prefetch = True
    #: gradients on ghost rows come home by the OWNER pulling them (plain peer loads + local reductions, the fast
    #: direction of the link) instead of the holder pushing remote reductions
    reverse_pull = True

    phase_events: list | None = None
    #: ``(velocities, masses, dt per system, batch_idx)`` of the owned atoms: when set (by ``DomainParallel`` for integrators
    #: whose closing update is the plain half kick) the kernel that collects the ghost copies' position gradients also
    #: writes the forces and applies ``v += dt/2 F/m`` (reverse halo fused with the integrator update)
    fused_finalize: tuple | None = None
    #: collect forces with the fused kernel (one thread per owned atom, copies in CSR form) instead of pull-add + negate
    fused_force_return: bool = True
    #: let the first kernel of the neighbour build fetch the ghost positions from their owners (no separate pull kernel);
    #: applies when the list is rebuilt every step (``neighbor_skin == 0``), else the pull kernel runs
    fold_ghost_pull: bool = True

    def __init__(self, wrapper: Any, config: Any, group: Any = None, max_neighbors: int | None = None) -> None:
        self.wrapper, self.model, self.config = wrapper, wrapper.model, config
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.cutoff = float(self.model.r_max)
        self.neighbor_skin = float(config.neighbor_skin)
        self.max_neighbors = max_neighbors or _nb.estimate_max_neighbors(self.cutoff + self.neighbor_skin)
        self.p2p: Any = None
        self.cap_rows = 0
        self._caps: dict[str, int] = {}
        self._bound: tuple[int, int] | None = None
        self.n_owned = self.n_ghost = 0
        self._nl: tuple | None = None
        self._nl_ref: torch.Tensor | None = None
        self._csr: Any = None
        self.num_list_builds = 0
        self.last_stats: dict[str, int] = {}

    # ------------------------------------------------------------------ dd view consumed by ``native.forward``
    @property
    def n_local(self) -> int:
        return self.n_owned + self.n_ghost

    @property
    def gpos(self) -> torch.Tensor:
        return self.gpos_buf

    def feature_buffer(self, key: str, shape: tuple[int, ...]) -> tuple[torch.Tensor, torch.Tensor]:
        buf, ptrs = self.feat[key]
        return buf[: shape[0]], ptrs

    def barrier(self) -> None:
        self.p2p.barrier()

    # ------------------------------------------------------------------ capacity / plan
    def _ensure_capacity(self, device: torch.device) -> None:
        """Row capacity agreed over the ranks (grow-only, bucketed); a new arena is a collective allocation."""
        from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

        with cap_agreement_group(self.group, device):
            cap = resolve_cap(self._caps, "rows", self.n_owned + self.n_ghost, initial_factor=1.2, stride=1024)
        if self.p2p is not None and cap <= self.cap_rows:
            return
        self.cap_rows = cap
        cfg = self.model.config
        C = cfg.channels
        widths = [sum(2 * l + 1 for l in ip.l_in) for ip in self.model.interactions]
        floats = cap * (3 + 3 + sum(w * C for w in widths) + sum(w * C for w in widths[1:]))
        self.p2p = None  # release the previous arena before asking for a larger one
        self.p2p = P2PContext(4 * floats + cap + 256 * (5 + 2 * len(widths)) + (1 << 16), device, self.group)
        a = self.p2p.arena
        self.pos_buf, self.pos_ptrs = a.alloc((cap, 3))
        self.gpos_buf, self.gpos_ptrs = a.alloc((cap, 3))
        self.used_buf, self.used_ptrs = a.alloc((cap,), torch.uint8)
        self.feat = {}
        for li, w in enumerate(widths):
            self.feat[f"u{li}"] = a.alloc((cap, w, C))
            if li > 0:
                self.feat[f"du{li}"] = a.alloc((cap, w, C))

    def _bind(self, sharded: Any) -> None:
        halo = sharded.halo
        key = (id(sharded), halo.num_builds)
        if key == self._bound:
            return
        owned = sharded.owned
        dev = owned.positions.device
        self.n_owned, self.n_ghost = sharded.n_owned, halo.n_ghost
        self._ensure_capacity(dev)
        n, ng = self.n_owned, self.n_ghost
        tables = build_pull_tables(sharded)
        self.ghost_home_rank, self.ghost_home_row = tables["home_rank"], tables["home_row"]
        self.ghost_image, self.wrap_image = tables["ghost_image"], tables["wrap_image"]
        self.ghost_shift = torch.empty(ng, 3, dtype=torch.float32, device=dev)
        z_owned = owned.atomic_numbers
        z_ghost = sharded._ghost_static[id(halo)]["atomic_numbers"]
        self.species = self.model.species_index(z_owned)
        self.species_local = torch.cat([self.species, self.model.species_index(z_ghost)]).contiguous()
        self.batch_idx = torch.zeros(n + ng, dtype=torch.int32, device=dev)
        self.batch_ptr = torch.tensor([0, n + ng], dtype=torch.int32, device=dev)
        self.batch_long = torch.zeros(n + ng, dtype=torch.long, device=dev)
        self.pbc = halo.local_pbc.reshape(1, 3).to(dev)
        self.ghost_used = self.used_buf[:ng]  # in the arena: owners read their copies' flags on the reverse path
        self.ghost_used.zero_()
        self.send_row, self.send_peer = tables["send_row"], tables["send_peer"]
        self.send_used_index, self.send_peer_row = tables["send_used_index"], tables["send_peer_row"]
        # the same send entries grouped by owned row (CSR): the fused force return reads every copy of a row in one thread
        order = torch.argsort(self.send_row.long(), stable=True)
        self.copy_peer = self.send_peer[order].contiguous()
        self.copy_row = self.send_peer_row[order].to(torch.int32).contiguous()
        self.copy_used_index = self.send_used_index[order].to(torch.int32).contiguous()
        self.copy_ptr = torch.zeros(n + 1, dtype=torch.int32, device=dev)
        torch.cumsum(torch.bincount(self.send_row.long(), minlength=n), 0, out=self.copy_ptr[1:])
        self._nl = self._nl_ref = self._csr = None
        self._sums = torch.zeros(10, dtype=torch.float64, device=dev)
        self._bound = key

    # ------------------------------------------------------------------ neighbour list over owned + ghost rows
    def _neighbors(self, pos_local: torch.Tensor, cell: torch.Tensor, ghost_pull: tuple | None = None) -> Any:
        from nvalchemi_toolkit_b200.models.mace import native

        n, n_local = self.n_owned, pos_local.shape[0]
        skin = self.neighbor_skin
        if self._csr is not None and skin > 0.0:
            moved = (pos_local - self._nl_ref).pow(2).sum(-1).max() > (0.5 * skin) ** 2
            if not bool(moved):  # one host read per step: the price of a list that is reused
                return self._csr
        k = self.max_neighbors
        while True:
            if self._nl is None or self._nl[0].shape != (n, k):
                self._nl = (torch.empty(n, k, dtype=torch.int32, device=pos_local.device),
                            torch.empty(n, dtype=torch.int32, device=pos_local.device),
                            torch.empty(n, k, 3, dtype=torch.int32, device=pos_local.device))
            nm, num, sh = _nb.neighbor_matrix(pos_local, cell, self.pbc, self.batch_idx, self.batch_ptr, self.cutoff + skin, k,
                                              False, out=self._nl, num_rows=n, ghost_pull=ghost_pull)
            csr = native.build_csr(nm, num, sh)
            if csr.max_count <= k:
                break
            k = self.max_neighbors = ((int(csr.max_count * 1.25) + 15) // 16) * 16
        self.ghost_used.zero_()
        _nops.mark_used_senders(csr.esend, csr.num_edges, n, self.ghost_used)
        self._csr = csr
        self._nl_ref = pos_local.clone() if skin > 0.0 else None
        self.num_list_builds += 1
        return csr

    # ------------------------------------------------------------------ one evaluation
    def forward(self, sharded: Any, active: set[str]) -> dict[str, torch.Tensor | None]:
        from nvalchemi_toolkit_b200.models.mace import native

        self._bind(sharded)
        owned = sharded.owned
        n, ng = self.n_owned, self.n_ghost
        mark = self._mark
        mark("bind")
        cell = owned.cell.reshape(3, 3).to(torch.float32)
        # owned positions in this rank's frame; ghost images relative to the owners' frames
        torch.addmm(owned.positions.detach(), self.wrap_image, cell, out=self.pos_buf[:n])
        if ng:
            torch.matmul(self.ghost_image, cell, out=self.ghost_shift)
        self.p2p.barrier()  # every rank's owned rows are in place (and last step's readers are done)
        pos_local = self.pos_buf[: n + ng]
        cell3 = cell.reshape(1, 3, 3).contiguous()
        fold = self.fold_ghost_pull and self.neighbor_skin == 0.0 and ng > 0
        if not fold:
            _nops.halo_pull_rows(self.pos_buf, n, self.ghost_home_rank, self.ghost_home_row, self.ghost_shift, self.pos_ptrs)
        mark("ghost_positions")
        # (with `fold` the first kernel of the neighbour build fetches the ghost positions from their owners itself)
        csr = self._neighbors(pos_local, cell3, (n, self.ghost_home_rank, self.ghost_home_row, self.ghost_shift, self.pos_ptrs)
                              if fold else None)
        mark("neighbor_list")
        want_f, want_s = "forces" in active, "stress" in active
        out = native.forward(self.model, {"positions": pos_local, "cell": cell3, "_csr": csr}, self.species,
                             self.batch_long, 1, want_f or want_s, want_s, dd=self)
        mark("model")
        sums = self._sums
        sums.zero_()
        sums[0:1] = out["energy"].double()
        if want_s:
            sums[1:10] = out["virial"].double().reshape(9)
        dist.all_reduce(sums, group=self.group)
        res: dict[str, torch.Tensor | None] = {"energy": sums[0:1].to(torch.float32).reshape(1, 1).clone(),
                                                "atomic_energies": out["node_energy"]}
        if want_f:
            res["forces"] = out["forces"].clone()
        if want_s:
            vol = torch.linalg.det(cell.double()).abs()
            virial = sums[1:10].reshape(1, 3, 3)
            res["virial"] = virial.to(torch.float32)
            res["stress"] = (-virial / vol).to(torch.float32)
        self.last_stats = {"n_owned": n, "n_ghost": ng, "n_edges": csr.num_edges}
        mark("reduce_outputs")
        return res

    # ------------------------------------------------------------------ optional phase timing (CUDA events)
    def _mark(self, name: str) -> None:
        """With ``phase_events`` set to a list, records a CUDA event at the end of each phase of :meth:`forward`."""
        ev = self.phase_events
        if ev is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.append((name, e))

    def phase_times_ms(self) -> dict[str, float]:
        """Device time per phase and evaluation (a phase that occurs several times per evaluation is summed), averaged over
        the evaluations recorded since ``phase_events`` was set (synchronises)."""
        ev = self.phase_events or []
        torch.cuda.synchronize()
        tot: dict[str, float] = {}
        for (_, e0), (name, e1) in zip(ev[:-1], ev[1:]):
            if name == "bind":
                name = "outside_forward"  # from the end of one evaluation to the start of the next: integrator, hooks
            tot[name] = tot.get(name, 0.0) + e0.elapsed_time(e1)
        n_eval = max(1, sum(1 for name, _ in ev if name == "reduce_outputs"))
        return {k: v / n_eval for k, v in tot.items()}

    def status(self) -> int:
        """0 while every device-side rendezvous completed within its bounded wait (one host read)."""
        return 0 if self.p2p is None else self.p2p.status()

    def check(self) -> None:
        """Raise ``PeerFailure`` if a peer missed a device-side rendezvous (one host read)."""
        if self.p2p is not None:
            self.p2p.check(wait=True)
