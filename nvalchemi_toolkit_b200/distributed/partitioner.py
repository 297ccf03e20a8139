# SPDX-License-Identifier: Apache-2.0
"""Spatial partitioning of a periodic (or open) cell over a 3-D grid of ranks.

Reference: ``nvalchemi/distributed/partitioner.py:28-537``: the rank grid is the factorisation of the world size that
minimises the surface between sub-domains, atoms are assigned by fractional coordinates, and an atom keeps its owner
while it stays within ``hysteresis`` of the owner's box (PBC-aware), which avoids ping-pong migration."""
from __future__ import annotations

import itertools

import torch


def factor_grid(world: int, face: tuple[float, float, float], max_per_dim: tuple[int, int, int] | None = None
                ) -> tuple[int, int, int]:
    """``(gx, gy, gz)`` with ``gx*gy*gz == world`` minimising the total cut area for cell face distances ``face``."""
    best, best_cost = (world, 1, 1), float("inf")
    for gx in range(1, world + 1):
        if world % gx:
            continue
        for gy in range(1, world // gx + 1):
            if (world // gx) % gy:
                continue
            g = (gx, gy, world // (gx * gy))
            if max_per_dim is not None and any(g[d] > max_per_dim[d] for d in range(3)):
                continue
            # area of the cuts normal to d scales with the product of the other two extents
            cost = sum((g[d] - 1) * face[(d + 1) % 3] * face[(d + 2) % 3] for d in range(3))
            if cost < best_cost - 1e-12:
                best, best_cost = g, cost
    return best


class SpatialPartitioner:
    def __init__(self, cell: torch.Tensor, pbc: torch.Tensor, world_size: int, cutoff: float,
                 grid_dims: tuple[int, int, int] | None = None, hysteresis: float = 0.0) -> None:
        self.world_size, self.cutoff, self.hysteresis = world_size, float(cutoff), float(hysteresis)
        self.update_cell(cell)
        self.pbc = pbc.reshape(3).bool().cpu()
        max_per = tuple(max(1, int(self.face[d] // cutoff)) for d in range(3))
        self.grid = tuple(grid_dims) if grid_dims is not None else factor_grid(world_size, tuple(self.face), max_per)
        if self.grid[0] * self.grid[1] * self.grid[2] != world_size:
            raise ValueError(f"rank grid {self.grid} does not match world size {world_size}")

    def update_cell(self, cell: torch.Tensor) -> None:
        self.cell = cell.reshape(3, 3).detach().double().cpu()
        self.inv = torch.linalg.inv(self.cell)
        self.face = [1.0 / float(self.inv[:, d].norm()) for d in range(3)]  # distance between opposite faces

    @property
    def cells_per_dim(self) -> tuple[int, int, int]:
        return tuple(max(1, int(self.face[d] // self.cutoff)) for d in range(3))

    def rank_coords(self, rank: int) -> tuple[int, int, int]:
        gx, gy, gz = self.grid
        return rank // (gy * gz), (rank // gz) % gy, rank % gz

    def rank_of(self, coords: torch.Tensor) -> torch.Tensor:
        gx, gy, gz = self.grid
        return (coords[..., 0] * gy + coords[..., 1]) * gz + coords[..., 2]

    def fractional(self, positions: torch.Tensor) -> torch.Tensor:
        return positions.double() @ self.inv.to(positions.device)

    def assign_atoms_to_ranks(self, positions: torch.Tensor) -> torch.Tensor:
        """Owner rank per atom from wrapped fractional coordinates (open dimensions are clamped)."""
        f = self.fractional(positions)
        pbc = self.pbc.to(positions.device)
        f = torch.where(pbc, f - torch.floor(f), f.clamp(0.0, 1.0 - 1e-12))
        g = torch.tensor(self.grid, device=positions.device)
        c = torch.minimum((f * g).long(), g - 1).clamp_min(0)
        return self.rank_of(c)

    def box(self, rank: int) -> tuple[torch.Tensor, torch.Tensor]:
        c = torch.tensor(self.rank_coords(rank), dtype=torch.float64)
        g = torch.tensor(self.grid, dtype=torch.float64)
        return c / g, (c + 1) / g

    def keeps_owner(self, positions: torch.Tensor, owner: torch.Tensor) -> torch.Tensor:
        """True where an atom is still inside its owner's box enlarged by the hysteresis band."""
        f = self.fractional(positions)
        g = torch.tensor(self.grid, dtype=torch.float64, device=positions.device)
        gy, gz = self.grid[1], self.grid[2]
        coords = torch.stack([owner // (gy * gz), (owner // gz) % gy, owner % gz], dim=-1).double()
        lo, hi = coords / g, (coords + 1) / g
        band = torch.tensor([self.hysteresis / self.face[d] for d in range(3)], dtype=torch.float64, device=positions.device)
        pbc = self.pbc.to(positions.device)
        centre = 0.5 * (lo + hi)
        d = f - centre
        d = torch.where(pbc, d - torch.round(d), d)  # minimum image relative to the box centre
        half = 0.5 * (hi - lo) + band
        return (d.abs() <= half).all(dim=-1)

    def neighbor_ranks(self, rank: int) -> list[int]:
        """Ranks whose boxes touch this rank's box (at most 26, fewer on small grids or open boundaries)."""
        c = self.rank_coords(rank)
        out = set()
        for off in itertools.product((-1, 0, 1), repeat=3):
            if off == (0, 0, 0):
                continue
            n = []
            for d in range(3):
                v = c[d] + off[d]
                if v < 0 or v >= self.grid[d]:
                    if not bool(self.pbc[d]):
                        break
                    v %= self.grid[d]
                n.append(v)
            else:
                r = (n[0] * self.grid[1] + n[1]) * self.grid[2] + n[2]
                if r != rank:
                    out.add(r)
        return sorted(out)


class IndexPartitioner:
    """Balanced contiguous index blocks (graph-partition strategy: geometry replicated, nodes split)."""

    def __init__(self, num_nodes: int, world_size: int) -> None:
        base, rem = divmod(num_nodes, world_size)
        self.bounds = [0]
        for r in range(world_size):
            self.bounds.append(self.bounds[-1] + base + (1 if r < rem else 0))

    def block(self, rank: int) -> tuple[int, int]:
        return self.bounds[rank], self.bounds[rank + 1]

    def owner(self, index: torch.Tensor) -> torch.Tensor:
        b = torch.tensor(self.bounds[1:], device=index.device)
        return torch.searchsorted(b, index, right=True)
