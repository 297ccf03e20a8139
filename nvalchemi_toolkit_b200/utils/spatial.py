# SPDX-License-Identifier: Apache-2.0
"""Spatial ordering of atoms for cache locality.

Message-passing kernels gather neighbour rows from global memory; when atoms that are close in space are also close
in memory, those gathers hit in L2 instead of going to HBM.  :func:`morton_order` returns the permutation that sorts
atoms along a Z-order curve over bins of about one neighbour shell; :func:`reorder_batch` applies a permutation to
every per-atom field of a single-system batch.
"""
from __future__ import annotations

import torch


def _spread_bits(v: torch.Tensor) -> torch.Tensor:
    """Insert two zero bits after each of the low 10 bits of ``v`` (int64)."""
    v = v & 0x3FF
    v = (v | (v << 16)) & 0x30000FF
    v = (v | (v << 8)) & 0x300F00F
    v = (v | (v << 4)) & 0x30C30C3
    v = (v | (v << 2)) & 0x9249249
    return v


def morton_order(positions: torch.Tensor, cell: torch.Tensor, bin_size: float = 4.0) -> torch.Tensor:
    """Permutation that sorts atoms by the Morton code of their bin (fractional coordinates, up to 1024 bins per axis)."""
    cell = cell.reshape(3, 3).to(positions.dtype)
    frac = positions @ torch.linalg.inv(cell)
    frac = frac - torch.floor(frac)
    nbins = torch.clamp((cell.norm(dim=1) / bin_size).floor(), 1, 1024).long()
    idx = torch.minimum((frac * nbins.to(frac.dtype)).long(), nbins - 1)
    code = _spread_bits(idx[:, 0]) | (_spread_bits(idx[:, 1]) << 1) | (_spread_bits(idx[:, 2]) << 2)
    return torch.argsort(code, stable=True)


def reorder_batch(batch: "object", perm: torch.Tensor) -> None:
    """Permute every per-atom field of a single-system batch in place (neighbour data must be rebuilt afterwards)."""
    if batch.num_graphs != 1:
        raise ValueError("reorder_batch handles one system; reorder each system before batching")
    group = batch._atoms_group
    for key in list(group.keys()):
        if key in ("neighbor_matrix", "num_neighbors", "neighbor_matrix_shifts"):
            del group.data[key]
            continue
        value = group[key]
        value.copy_(value[perm])
