# SPDX-License-Identifier: Apache-2.0
"""Builders shared by tests."""
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch


def random_molecule(n: int, seed: int, n_edges: int = 0, periodic: bool = False, dtype=torch.float32) -> AtomicData:
    g = torch.Generator().manual_seed(seed)
    kw = dict(atomic_numbers=torch.tensor([1, 6, 7, 8])[torch.randint(0, 4, (n,), generator=g)],
              positions=(torch.rand(n, 3, generator=g) * 10).to(dtype), forces=torch.zeros(n, 3, dtype=dtype),
              energy=torch.zeros(1, 1, dtype=dtype))
    if n_edges:
        kw["neighbor_list"] = torch.randint(0, n, (n_edges, 2), generator=g)
        kw["shifts"] = torch.zeros(n_edges, 3, dtype=dtype)
    if periodic:
        kw["cell"] = (torch.eye(3) * 10).to(dtype)
        kw["pbc"] = torch.tensor([True, True, True])
    return AtomicData(**kw)


def random_batch(sizes, seed: int = 0, n_edges: int = 0, periodic: bool = False, device="cpu", dtype=torch.float32) -> Batch:
    data = [random_molecule(n, seed + i, n_edges, periodic, dtype) for i, n in enumerate(sizes)]
    return Batch.from_data_list(data, device=device)


def fcc_supercell(n_cells: int, a: float = 3.61, z: int = 29, noise: float = 0.05, seed: int = 0,
                  dtype=torch.float32) -> AtomicData:
    g = torch.Generator().manual_seed(seed)
    base = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]], dtype=torch.float64)
    r = torch.arange(n_cells, dtype=torch.float64)
    grid = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 1, 3)
    pos = ((grid + base[None]).reshape(-1, 3) * a)
    pos = pos + noise * torch.randn(pos.shape, generator=g, dtype=torch.float64)
    n = pos.shape[0]
    return AtomicData(atomic_numbers=torch.full((n,), z), positions=pos.to(dtype), cell=(torch.eye(3) * a * n_cells).to(dtype),
                      pbc=torch.tensor([True, True, True]), forces=torch.zeros(n, 3, dtype=dtype),
                      energy=torch.zeros(1, 1, dtype=dtype))
