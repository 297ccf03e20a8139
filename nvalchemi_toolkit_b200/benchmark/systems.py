# SPDX-License-Identifier: Apache-2.0
"""Synthetic benchmark systems (reference ``benchmark/distributed/_benchmark_common.py:71-620``): argon cluster, bcc iron,
rock-salt NaCl, a beta-cristobalite-like SiO2 framework and a methane box, each scalable by repetition count."""
from __future__ import annotations

import math
from typing import Any, Callable

import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch


def _crystal(basis: torch.Tensor, numbers: torch.Tensor, a: float, reps: tuple[int, int, int], noise: float, seed: int,
             dtype: torch.dtype, charges: torch.Tensor | None = None) -> AtomicData:
    g = torch.Generator().manual_seed(seed)
    rx, ry, rz = (torch.arange(r, dtype=torch.float64) for r in reps)
    grid = torch.stack(torch.meshgrid(rx, ry, rz, indexing="ij"), -1).reshape(-1, 1, 3)
    pos = ((grid + basis[None].double()).reshape(-1, 3) * a)
    pos = pos + noise * torch.randn(pos.shape, generator=g, dtype=torch.float64)
    z = numbers.repeat(grid.shape[0])
    n = pos.shape[0]
    kw: dict[str, Any] = dict(atomic_numbers=z, positions=pos.to(dtype), cell=(torch.diag(torch.tensor(reps, dtype=torch.float64)) * a).to(dtype),
                              pbc=torch.tensor([True, True, True]), forces=torch.zeros(n, 3, dtype=dtype),
                              energy=torch.zeros(1, 1, dtype=dtype), velocities=torch.zeros(n, 3, dtype=dtype))
    data = AtomicData(**kw)
    if charges is not None:
        data.__dict__["node_charges"] = charges.repeat(grid.shape[0]).to(dtype)
    return data


def fcc(reps: int, a: float = 3.61, z: int = 29, **kw: Any) -> AtomicData:
    basis = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]])
    return _crystal(basis, torch.full((4,), z), a, (reps,) * 3, kw.get("noise", 0.05), kw.get("seed", 0), kw.get("dtype", torch.float32))


def bcc_iron(reps: int, a: float = 2.87, **kw: Any) -> AtomicData:
    basis = torch.tensor([[0, 0, 0], [0.5, 0.5, 0.5]])
    return _crystal(basis, torch.full((2,), 26), a, (reps,) * 3, kw.get("noise", 0.03), kw.get("seed", 0), kw.get("dtype", torch.float32))


def nacl(reps: int, a: float = 5.64, **kw: Any) -> AtomicData:
    basis = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5],
                          [0.5, 0, 0], [0, 0.5, 0], [0, 0, 0.5], [0.5, 0.5, 0.5]])
    z = torch.tensor([11] * 4 + [17] * 4)
    q = torch.tensor([1.0] * 4 + [-1.0] * 4)
    return _crystal(basis, z, a, (reps,) * 3, kw.get("noise", 0.03), kw.get("seed", 0), kw.get("dtype", torch.float32), charges=q)


def silica(reps: int, a: float = 7.16, **kw: Any) -> AtomicData:
    """Idealised beta-cristobalite: Si on a diamond lattice, O at the Si-Si bond midpoints (24 atoms per cell)."""
    fcc_b = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]])
    si = torch.cat([fcc_b, fcc_b + 0.25])
    bonds = torch.tensor([[1, 1, 1], [1, -1, -1], [-1, 1, -1], [-1, -1, 1]]) * 0.125
    o = (fcc_b[:, None, :] + bonds[None]).reshape(-1, 3) % 1.0
    basis = torch.cat([si, o])
    z = torch.tensor([14] * 8 + [8] * 16)
    q = torch.tensor([2.4] * 8 + [-1.2] * 16)
    return _crystal(basis, z, a, (reps,) * 3, kw.get("noise", 0.02), kw.get("seed", 0), kw.get("dtype", torch.float32), charges=q)


def argon_cluster(n_atoms: int, spacing: float = 3.8, **kw: Any) -> AtomicData:
    """Roughly spherical open-boundary cluster cut from an fcc lattice."""
    dtype = kw.get("dtype", torch.float32)
    reps = int((n_atoms / 4) ** (1 / 3)) + 3
    d = fcc(reps, a=spacing * 2 ** 0.5, z=18, noise=kw.get("noise", 0.02), seed=kw.get("seed", 0), dtype=torch.float64)
    centre = d.positions.mean(0)
    keep = torch.argsort((d.positions - centre).norm(dim=-1))[:n_atoms]
    pos = d.positions[keep] - centre
    box = float(pos.abs().max()) * 2 + 20.0
    return AtomicData(atomic_numbers=torch.full((n_atoms,), 18), positions=(pos + box / 2).to(dtype),
                      cell=(torch.eye(3) * box).to(dtype), pbc=torch.tensor([False, False, False]),
                      forces=torch.zeros(n_atoms, 3, dtype=dtype), energy=torch.zeros(1, 1, dtype=dtype),
                      velocities=torch.zeros(n_atoms, 3, dtype=dtype))


def methane_box(reps: int, spacing: float = 4.2, **kw: Any) -> AtomicData:
    """Methane molecules on a simple cubic lattice with alternating orientation."""
    d = 1.09 / 3 ** 0.5 / spacing
    h = torch.tensor([[1, 1, 1], [1, -1, -1], [-1, 1, -1], [-1, -1, 1]]) * d
    basis = torch.cat([torch.full((1, 3), 0.5), 0.5 + h])
    return _crystal(basis, torch.tensor([6, 1, 1, 1, 1]), spacing, (reps,) * 3, kw.get("noise", 0.01), kw.get("seed", 0),
                    kw.get("dtype", torch.float32))


def water_box(n_molecules: int, density: float = 1.0, seed: int = 0, dtype: torch.dtype = torch.float32, **kw: Any) -> AtomicData:
    """Periodic box of ``n_molecules`` rigid-geometry water molecules at ``density`` g/cm^3: oxygens on a jittered simple
    cubic lattice (the ``ceil(n^(1/3))^3`` sites are subsampled), O-H 0.96 A, H-O-H 104.5 degrees, uniformly random
    orientations, partial charges O -0.82 / H +0.41 (the ``charges`` field)."""
    g = torch.Generator().manual_seed(seed)
    vol = n_molecules * 18.015 / (density * 0.602214)          # A^3: 18.015 g/mol over N_A * 1e-24 cm^3
    box = vol ** (1.0 / 3.0)
    m = int(math.ceil(n_molecules ** (1.0 / 3.0) - 1e-9))
    sites = torch.stack(torch.meshgrid(*(torch.arange(m, dtype=torch.float64),) * 3, indexing="ij"), -1).reshape(-1, 3)
    pick = torch.randperm(sites.shape[0], generator=g)[:n_molecules]
    o = (sites[pick] + 0.5 + 0.15 * (torch.rand(n_molecules, 3, generator=g, dtype=torch.float64) - 0.5)) * (box / m)
    # random rotations from normalised quaternions
    q = torch.randn(n_molecules, 4, generator=g, dtype=torch.float64)
    q = q / q.norm(dim=1, keepdim=True)
    w, x, y, z = q.unbind(1)
    rot = torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w),
                       2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w),
                       2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], 1).reshape(-1, 3, 3)
    half = math.radians(104.5) / 2.0
    h_local = 0.96 * torch.tensor([[math.sin(half), 0.0, math.cos(half)], [-math.sin(half), 0.0, math.cos(half)]], dtype=torch.float64)
    h = o[:, None, :] + torch.einsum("nij,kj->nki", rot, h_local)
    pos = torch.cat([o[:, None, :], h], 1).reshape(-1, 3)
    n = pos.shape[0]
    data = AtomicData(atomic_numbers=torch.tensor([8, 1, 1]).repeat(n_molecules), positions=pos.to(dtype),
                      cell=(torch.eye(3, dtype=torch.float64) * box).to(dtype), pbc=torch.tensor([True, True, True]),
                      forces=torch.zeros(n, 3, dtype=dtype), energy=torch.zeros(1, 1, dtype=dtype),
                      velocities=torch.zeros(n, 3, dtype=dtype),
                      charges=torch.tensor([-0.82, 0.41, 0.41]).repeat(n_molecules).to(dtype))
    return data


SYSTEMS: dict[str, Callable[..., AtomicData]] = {"fcc_cu": fcc, "bcc_fe": bcc_iron, "nacl": nacl, "sio2": silica,
                                                 "ar_cluster": argon_cluster, "ch4": methane_box, "water": water_box}


def build(name: str, size: int, device: str | torch.device = "cpu", **kw: Any) -> Batch:
    data = SYSTEMS[name](size, **kw)
    batch = Batch.from_data_list([data], device=device)
    q = data.__dict__.get("node_charges")
    if q is not None:
        batch.add_key("node_charges", q.to(device), level="node", overwrite=True)
    return batch
