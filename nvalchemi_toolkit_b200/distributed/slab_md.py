# SPDX-License-Identifier: Apache-2.0
"""Domain-decomposed MD of one large periodic system with the native MACE: slabs along one cell axis, one per GPU.

What the reference does with ``DomainParallel`` + ``HaloStrategy`` + ShardTensor dispatch
(``nvalchemi/distributed/domain_parallel.py:251-485``, ``distributed/strategy.py:680-911``) is done here with explicit
kernels over peer-mapped memory:

* **topology** (rare): owned atoms of all ranks are all-gathered (NCCL), every rank derives the same slab ownership,
  spatial ordering and ghost lists; ghosts are the atoms (and periodic images) within ``cutoff + halo_skin`` of the
  rank's slab; each ghost records its owner rank, its row there and its image shift;
* **per step**: the consumer *pulls* ghost positions from the owners' position buffers (P2P loads), builds the
  neighbour list over owned + ghost atoms, and evaluates MACE on its owned atoms.  Sender features of ghosts are
  gathered from the owner inside the convolution kernels; the adjoint pushes feature and position gradients of ghosts to
  their owners with reductions over NVLink.  Device-side flag barriers separate the phases.  Each edge is evaluated
  exactly once (at the rank owning its receiver), energies are sums over owned atoms;
* the topology is rebuilt (with migration of atoms that left their slab) when some atom has moved more than
  ``halo_skin / 2`` since the last build; the decision uses the flag of the previous step so that no step waits on
  the host.
"""
from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import KB_EV, fs_to_internal_time, per_fs_to_internal_rate
from nvalchemi_toolkit_b200.models.mace import native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops
from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext


class _DDView:
    """What ``native.forward`` needs to know about the decomposition."""

    def __init__(self, owner: "SlabDomainMD") -> None:
        self.o = owner

    @property
    def n_owned(self) -> int:
        return self.o.n_owned

    @property
    def home_rank(self) -> torch.Tensor:
        return self.o.home_rank

    @property
    def home_row(self) -> torch.Tensor:
        return self.o.home_row

    @property
    def gpos(self) -> torch.Tensor:
        return self.o.gpos

    @property
    def gpos_ptrs(self) -> torch.Tensor:
        return self.o.gpos_ptrs

    #: ghost rows of node features are copied from their owners once per layer (bulk pull at NVLink bandwidth) and ghost
    #: rows of the gradients are returned once per layer (bulk push); with False the convolution kernels touch peer
    #: memory per edge instead
    prefetch = True

    @property
    def n_local(self) -> int:
        return self.o.n_owned + self.o.n_ghost

    @property
    def ghost_home_rank(self) -> torch.Tensor:
        return self.o.ghost_home_rank

    @property
    def species_local(self) -> torch.Tensor:
        """Species index of owned and ghost rows (the first interaction reads a per-species feature table)."""
        return self.o.species_local

    @property
    def ghost_home_row(self) -> torch.Tensor:
        return self.o.ghost_home_row

    def feature_buffer(self, key: str, shape: tuple[int, ...]) -> tuple[torch.Tensor, torch.Tensor]:
        buf, ptrs = self.o.feat[key]
        n = shape[0]
        return buf[:n], ptrs

    def barrier(self) -> None:
        self.o.p2p.barrier()


class SlabDomainMD:
    """NVT-Langevin (or NVE when ``friction`` is None) MD of a periodic system decomposed into slabs."""

    def __init__(self, model: Any, cell: torch.Tensor, n_total: int, device: torch.device, dt: float = 1.0,
                 temperature: float = 300.0, friction: float | None = 0.01, seed: int = 7, halo_skin: float = 1.0,
                 max_neighbors: int = 64, axis: int = 0, group: dist.ProcessGroup | None = None) -> None:
        self.model = model
        self.cfg = model.config
        self.device = device
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.cell = cell.to(device=device, dtype=torch.float32).reshape(3, 3).contiguous()
        self.inv = torch.linalg.inv(self.cell.double())
        self.axis = axis
        self.n_total = int(n_total)
        self.cutoff = float(self.cfg.r_max)
        self.halo_skin = float(halo_skin)
        self.max_neighbors = max_neighbors
        self.dt = torch.tensor([fs_to_internal_time(dt)], device=device)
        self.kT = torch.tensor([temperature * KB_EV], device=device)
        self.gamma = None if friction is None else torch.tensor([per_fs_to_internal_rate(friction)], device=device)
        self.seed = seed
        self.step_count = 0
        face = 1.0 / float(self.inv[:, axis].norm())
        self.h_frac = (self.cutoff + self.halo_skin) / face
        if self.h_frac * self.world > 1.0 + 1e-9 and self.world > 1:
            raise ValueError("slabs are thinner than the halo; use fewer ranks or a larger cell")
        C = self.cfg.channels
        nlm_hidden = (self.cfg.hidden_lmax + 1) ** 2
        density_rows = self.n_total / self.world
        self.cap_owned = int(density_rows * 1.15) + 4096
        ghost_est = 2.0 * self.h_frac * self.n_total
        self.cap_local = self.cap_owned + int(ghost_est * 1.3) + 4096
        nbytes = 4 * (3 * self.cap_local + 3 * self.cap_local + self.cap_local * C * (1 + 2 * nlm_hidden)) + (1 << 16)
        self.p2p = P2PContext(nbytes, device, self.group)
        a = self.p2p.arena
        self.pos_buf, self.pos_ptrs = a.alloc((self.cap_local, 3))
        # row capacity = owned + ghost: owners keep their rows at the front (peers address them by owner row), ghost rows
        # behind them hold the copies pulled from / the gradients to be pushed to the owners
        self.gpos_buf, self.gpos_ptrs = a.alloc((self.cap_local, 3))
        self.feat = {"u0": a.alloc((self.cap_local, 1, C)), "u1": a.alloc((self.cap_local, nlm_hidden, C)),
                     "du1": a.alloc((self.cap_local, nlm_hidden, C))}
        self.view = _DDView(self)
        self.n_owned = 0
        self.n_ghost = 0
        self._flag_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._flag_event: torch.cuda.Event | None = None
        self.num_topology_builds = 0
        self.last_energy_local: torch.Tensor | None = None

    # ------------------------------------------------------------------ state
    @property
    def pos(self) -> torch.Tensor:
        return self.pos_buf[: self.n_owned]

    @property
    def gpos(self) -> torch.Tensor:
        return self.gpos_buf

    def set_owned(self, pos: torch.Tensor, vel: torch.Tensor, mass: torch.Tensor, z: torch.Tensor, gid: torch.Tensor
                  ) -> None:
        """Install this rank's current atoms (any subset; ownership is re-derived) and build the topology."""
        self._owned = {"pos": pos.to(self.device, torch.float32), "vel": vel.to(self.device, torch.float32),
                       "mass": mass.to(self.device, torch.float32), "z": z.to(self.device).long(),
                       "gid": gid.to(self.device).long()}
        self.rebuild_topology()
        self.compute_forces()

    def _gather_all(self, t: torch.Tensor, counts: list[int]) -> torch.Tensor:
        mx = max(counts)
        pad = t.new_zeros((mx,) + tuple(t.shape[1:]))
        pad[: t.shape[0]] = t
        out = t.new_empty((self.world * mx,) + tuple(t.shape[1:]))
        dist.all_gather_into_tensor(out, pad, group=self.group)
        out = out.reshape(self.world, mx, *t.shape[1:])
        return torch.cat([out[r, : counts[r]] for r in range(self.world)], dim=0)

    def rebuild_topology(self) -> None:
        """All-gather owned atoms, re-derive ownership (migration), spatial order and ghost lists."""
        st = self._owned
        if self.n_owned:
            st["pos"] = self.pos.clone()
        n_mine = torch.tensor([st["pos"].shape[0]], device=self.device)
        counts_t = torch.empty(self.world, dtype=n_mine.dtype, device=self.device)
        dist.all_gather_into_tensor(counts_t, n_mine, group=self.group)
        counts = [int(c) for c in counts_t.tolist()]
        fl = torch.cat([st["pos"], st["vel"], st["mass"].unsqueeze(1), st["z"].float().unsqueeze(1)], dim=1)
        fl = self._gather_all(fl, counts)
        gid = self._gather_all(st["gid"], counts)
        pos_all, vel_all, mass_all, z_all = fl[:, 0:3], fl[:, 3:6], fl[:, 6], fl[:, 7].long()
        frac = pos_all.double() @ self.inv
        frac = frac - torch.floor(frac)
        pos_w = (frac @ self.cell.double()).float()
        fx = frac[:, self.axis]
        W, rank = self.world, self.rank
        owner = torch.clamp((fx * W).long(), 0, W - 1)
        # spatial ordering: bins of ~cutoff, slab axis slowest so that consecutive rows are neighbours
        nb = [max(1, int(1.0 / float(self.inv[:, d].norm()) / self.cutoff)) for d in range(3)]
        other = [d for d in range(3) if d != self.axis]
        bx = torch.clamp((fx * nb[self.axis]).long(), 0, nb[self.axis] - 1)
        b1 = torch.clamp((frac[:, other[0]] * nb[other[0]]).long(), 0, nb[other[0]] - 1)
        b2 = torch.clamp((frac[:, other[1]] * nb[other[1]]).long(), 0, nb[other[1]] - 1)
        key = ((owner * nb[self.axis] + bx) * nb[other[0]] + b1) * nb[other[1]] + b2
        order = torch.argsort(key, stable=True)
        own_sorted = owner[order]
        start = torch.searchsorted(own_sorted, torch.arange(W + 1, device=self.device))
        row_in_owner = torch.empty_like(order)
        row_in_owner[order] = torch.arange(order.numel(), device=self.device) - start[own_sorted]
        mine = order[start[rank]: start[rank + 1]]
        n_owned = int(mine.numel())
        if n_owned > self.cap_owned:
            raise MemoryError("owned-atom capacity exceeded; load imbalance too large for the slab decomposition")
        lo, hi, h = rank / W, (rank + 1) / W, self.h_frac
        g_idx, g_shift = [], []
        for s in (-1, 0, 1):
            f2 = fx + s
            sel = (f2 >= lo - h) & (f2 < hi + h)
            if s == 0:
                sel &= owner != rank
            idx = torch.nonzero(sel).squeeze(1)
            g_idx.append(idx)
            g_shift.append(torch.full((idx.numel(),), float(s), device=self.device))
        g_idx, g_s = torch.cat(g_idx), torch.cat(g_shift)
        n_ghost = int(g_idx.numel())
        if n_owned + n_ghost > self.cap_local:
            raise MemoryError("ghost capacity exceeded")
        self.n_owned, self.n_ghost = n_owned, n_ghost
        self.vel = vel_all[mine].contiguous()
        self.mass = mass_all[mine].contiguous()
        self.z = z_all[mine].contiguous()
        self.gid = gid[mine].contiguous()
        self.species = self.model.species_index(self.z)
        self.species_local = torch.cat([self.species, self.model.species_index(z_all[g_idx])]).contiguous()
        self.pos_buf[:n_owned] = pos_w[mine]
        self.ref_pos = pos_w[mine].clone()
        self.forces = torch.zeros(n_owned, 3, device=self.device)
        self.ghost_shift = (g_s.unsqueeze(1) * self.cell[self.axis].unsqueeze(0)).contiguous()
        self.ghost_home_rank = owner[g_idx].to(torch.int32).contiguous()
        self.ghost_home_row = row_in_owner[g_idx].to(torch.int32).contiguous()
        self.home_rank = torch.cat([torch.full((n_owned,), rank, dtype=torch.int32, device=self.device),
                                    self.ghost_home_rank]).contiguous()
        self.home_row = torch.cat([torch.arange(n_owned, dtype=torch.int32, device=self.device),
                                   self.ghost_home_row]).contiguous()
        n_local = n_owned + n_ghost
        self.batch_idx = torch.zeros(n_local, dtype=torch.int32, device=self.device)
        self.batch_ptr = torch.tensor([0, n_local], dtype=torch.int32, device=self.device)
        self.owned_batch_idx = self.batch_idx[:n_owned]
        pbc = [True, True, True]
        pbc[self.axis] = False  # images along the slab axis are explicit ghost rows
        self.pbc = torch.tensor([pbc], device=self.device)
        self._nl = None
        self._owned = {"pos": None, "vel": self.vel, "mass": self.mass, "z": self.z, "gid": self.gid}
        self._flags = torch.zeros(1, dtype=torch.bool, device=self.device)
        self._flag_event = None
        self._flag_host.zero_()
        self.num_topology_builds += 1
        self.p2p.barrier()

    # ------------------------------------------------------------------ optional phase timing (CUDA events)
    def _phase(self, name: str) -> Any:
        import contextlib

        if not getattr(self, "profile", False):
            return contextlib.nullcontext()
        owner = self

        class _Timer:
            def __enter__(self) -> None:
                self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.a.record()

            def __exit__(self, *exc: Any) -> None:
                self.b.record()
                owner.__dict__.setdefault("_phase_events", {}).setdefault(name, []).append((self.a, self.b))

        return _Timer()

    def phase_summary(self) -> dict[str, float]:
        """Milliseconds per recorded occurrence of every phase (set ``self.profile = True`` before stepping)."""
        torch.cuda.synchronize(self.device)
        return {k: sum(a.elapsed_time(b) for a, b in v) / max(1, len(v)) for k, v in getattr(self, "_phase_events", {}).items()}

    # ------------------------------------------------------------------ one force evaluation
    def refresh_ghosts(self) -> None:
        self.p2p.barrier()  # every rank finished moving its owned atoms
        _nops.halo_pull_rows(self.pos_buf, self.n_owned, self.ghost_home_rank, self.ghost_home_row, self.ghost_shift,
                             self.pos_ptrs)

    def compute_forces(self) -> None:
        with self._phase("ghost_positions"):
            self.refresh_ghosts()
        n_local = self.n_owned + self.n_ghost
        pos_local = self.pos_buf[:n_local]
        cell = self.cell.reshape(1, 3, 3)
        k = self.max_neighbors
        with self._phase("neighbors"):
            while True:
                if self._nl is None or self._nl[0].shape != (n_local, k):
                    self._nl = (torch.empty(n_local, k, dtype=torch.int32, device=self.device),
                                torch.empty(n_local, dtype=torch.int32, device=self.device),
                                torch.empty(n_local, k, 3, dtype=torch.int32, device=self.device))
                nm, num, sh = _nb.neighbor_matrix(pos_local, cell, self.pbc, self.batch_idx, self.batch_ptr, self.cutoff, k,
                                                  False, out=self._nl)
                csr = native.build_csr(nm[: self.n_owned], num[: self.n_owned], sh[: self.n_owned])
                if csr.max_count <= k:
                    break
                k = self.max_neighbors = ((int(csr.max_count * 1.25) + 15) // 16) * 16
        data = {"positions": pos_local, "cell": cell, "_csr": csr}
        with self._phase("model"):
            out = native.forward(self.model, data, self.species, self.batch_idx.long(), 1, True, False, dd=self.view)
        self.forces = out["forces"]
        self.last_energy_local = out["energy"]

    # ------------------------------------------------------------------ MD step
    def _consume_rebuild_flag(self) -> bool:
        """Flag raised by the displacement check of the previous step (already reduced over ranks)."""
        if self._flag_event is None:
            return False
        self._flag_event.synchronize()
        return bool(self._flag_host.item())

    def step(self) -> None:
        if self._consume_rebuild_flag():
            self.rebuild_topology()
        pos = self.pos
        b = self.owned_batch_idx
        timer = self._phase("integrate_and_flags")
        timer.__enter__()
        if self.gamma is not None:
            _ops.langevin_half_step(pos, self.vel, self.forces, self.mass, self.dt, self.kT, self.gamma,
                                    self.seed + self.step_count, b, self.gid)
        else:
            _ops.vv_position_update(pos, self.vel, self.forces, self.mass, self.dt, b)
        # displacement check against the positions of the last topology build (consumed at the next step)
        self._flags.zero_()
        _ops.batch_neighbor_list_rebuild_inplace(self.ref_pos, pos, b, self._flags, 0.5 * self.halo_skin, False,
                                                 self.cell.reshape(1, 3, 3), self.inv.float().reshape(1, 3, 3).contiguous(),
                                                 torch.ones(1, 3, dtype=torch.bool, device=self.device))
        fl = self._flags.to(torch.int32)
        dist.all_reduce(fl, op=dist.ReduceOp.MAX, group=self.group)
        self._flag_host.copy_(fl, non_blocking=True)
        self._flag_event = torch.cuda.Event()
        self._flag_event.record()
        timer.__exit__(None, None, None)
        self.compute_forces()
        _ops.vv_velocity_finalize(self.vel, self.forces, self.mass, self.dt, b)
        self.step_count += 1

    def run(self, n_steps: int) -> None:
        for _ in range(n_steps):
            self.step()

    # ------------------------------------------------------------------ observables
    def energy(self) -> float:
        e = self.last_energy_local.double().clone()
        dist.all_reduce(e, group=self.group)
        return float(e)

    def kinetic_energy(self) -> float:
        ke = _ops.compute_kinetic_energy(self.vel, self.mass, self.owned_batch_idx, 1).double()
        dist.all_reduce(ke, group=self.group)
        return float(ke)

    def gather(self) -> dict[str, torch.Tensor]:
        """All atoms ordered by global id (every rank gets the result)."""
        counts_t = torch.empty(self.world, dtype=torch.long, device=self.device)
        dist.all_gather_into_tensor(counts_t, torch.tensor([self.n_owned], device=self.device), group=self.group)
        counts = [int(c) for c in counts_t.tolist()]
        fl = self._gather_all(torch.cat([self.pos, self.vel, self.forces], dim=1), counts)
        gid = self._gather_all(self.gid, counts)
        order = torch.argsort(gid)
        return {"positions": fl[order, 0:3], "velocities": fl[order, 3:6], "forces": fl[order, 6:9], "gid": gid[order]}

    # ------------------------------------------------------------------ benchmark helpers
    @classmethod
    def for_benchmark(cls, cells: int, device: torch.device, skin: float = 0.0, max_neighbors: int = 64,
                      halo_skin: float = 1.0, atom_order: str = "lattice") -> "SlabDomainMD":
        """fcc Cu supercell of ``cells^3`` conventional cells; every rank generates only its own slab."""
        from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig

        torch.manual_seed(0)
        cfg = MACEConfig(atomic_numbers=[29], r_max=5.0, num_bessel=8, num_polynomial_cutoff=5, max_ell=3,
                         num_interactions=2, channels=128, hidden_lmax=1, correlation=3, avg_num_neighbors=42.0)
        model = MACE(cfg).to(device)
        world, rank = dist.get_world_size(), dist.get_rank()
        a = 3.61
        cell = torch.eye(3) * a * cells
        sim = cls(model, cell, 4 * cells ** 3, device, dt=1.0, temperature=300.0, friction=0.01, seed=7,
                  halo_skin=halo_skin, max_neighbors=max_neighbors)
        x0, x1 = rank * cells // world, (rank + 1) * cells // world
        base = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]], device=device)
        rx = torch.arange(x0, x1, device=device, dtype=torch.float32)
        r = torch.arange(cells, device=device, dtype=torch.float32)
        grid = torch.stack(torch.meshgrid(rx, r, r, indexing="ij"), -1).reshape(-1, 1, 3)
        pos = ((grid + base[None]).reshape(-1, 3) * a)
        n = pos.shape[0]
        gid = torch.arange(n, device=device) + 4 * cells * cells * x0
        g = torch.Generator(device=device).manual_seed(1000 + rank)
        pos = pos + 0.05 * torch.randn(pos.shape, generator=g, device=device) + 0.01
        if atom_order == "morton":  # memory order along a Z-curve: neighbour gathers stay in L2
            from nvalchemi_toolkit_b200.utils.spatial import morton_order

            perm = morton_order(pos, cell.to(device), 4.0)
            pos, gid = pos[perm].contiguous(), gid[perm].contiguous()
        mass = torch.full((n,), 63.546, device=device)
        vel = torch.zeros_like(pos)
        _ops.initialize_velocities(vel, mass, 300.0, torch.zeros(n, dtype=torch.int32, device=device), random_seed=1,
                                   remove_com=False, rescale=False, atom_ids=gid)
        sim.set_owned(pos, vel, mass, torch.full((n,), 29, device=device), gid)
        return sim

    def e2e_bytes(self) -> tuple[int, int]:
        n = self.n_owned
        return (2 * n * 12, 2 * n * 12 + 4)

    def host_driven_step(self) -> float:
        """One step with the state owned by the host: positions/velocities in from pinned memory, results back."""
        n = self.n_owned
        if getattr(self, "_host", None) is None or self._host[0].shape[0] != n:
            self._host = (torch.empty(n, 3).pin_memory(), torch.empty(n, 3).pin_memory(), torch.empty(1).pin_memory())
            self._host[0].copy_(self.pos)
            self._host[1].copy_(self.vel)
        hp, hv, he = self._host
        self.pos.copy_(hp, non_blocking=True)
        self.vel.copy_(hv, non_blocking=True)
        self.step()
        if self.n_owned != n:  # topology rebuilt inside the step
            self._host = None
            return self.energy()
        hp.copy_(self.pos, non_blocking=True)
        hv.copy_(self.vel, non_blocking=True)
        e = self.last_energy_local.double().clone()
        dist.all_reduce(e, group=self.group)
        he.copy_(e.float(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(he)
