# SPDX-License-Identifier: Apache-2.0
"""Autograd helpers for conservative models: forces, strain trick, stresses.

Conventions (reference ``docs/userguide/about/conventions.md:9-41`` and
``nvalchemi/models/_utils.py:49-328``): virial ``W = -dE/d(strain)``, stress
``sigma = -W / V`` (tensile positive); the strain is a symmetric ``[B,3,3]`` tensor
applied as ``r -> r (1 + eps)`` and ``cell -> cell (1 + eps)``.
"""
from __future__ import annotations

import torch


def autograd_forces(energy: torch.Tensor, positions: torch.Tensor, training: bool = False) -> torch.Tensor:
    (g,) = torch.autograd.grad(energy.sum(), positions, create_graph=training, retain_graph=training)
    return -g


def prepare_strain(positions: torch.Tensor, cell: torch.Tensor, batch_idx: torch.Tensor
                   ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Return ``(strained_positions, strained_cell, strain)`` with ``strain`` requiring grad (zeros)."""
    b = cell.shape[0]
    strain = torch.zeros(b, 3, 3, dtype=positions.dtype, device=positions.device, requires_grad=True)
    sym = 0.5 * (strain + strain.transpose(-1, -2))
    eye = torch.eye(3, dtype=positions.dtype, device=positions.device)
    deform = eye + sym
    pos = torch.einsum("ni,nij->nj", positions, deform[batch_idx.long()])
    return pos, cell @ deform, strain


def autograd_stresses(energy: torch.Tensor, strain: torch.Tensor, cell: torch.Tensor, training: bool = False
                      ) -> torch.Tensor:
    (g,) = torch.autograd.grad(energy.sum(), strain, create_graph=training, retain_graph=training)
    vol = torch.linalg.det(cell).abs().clamp_min(1e-30)
    return g / vol[:, None, None]


def autograd_forces_and_stresses(energy: torch.Tensor, positions: torch.Tensor, strain: torch.Tensor,
                                 cell: torch.Tensor, training: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    gp, gs = torch.autograd.grad(energy.sum(), [positions, strain], create_graph=training, retain_graph=training)
    vol = torch.linalg.det(cell).abs().clamp_min(1e-30)
    return -gp, gs / vol[:, None, None]


def sum_outputs(*outs: dict, additive_keys: frozenset[str] = frozenset({"energy", "forces", "stress"})) -> dict:
    """Sum additive keys across model outputs; non-additive keys take the last non-None value."""
    result: dict = {}
    for o in outs:
        for k, v in o.items():
            if v is None:
                result.setdefault(k, None)
            elif k in additive_keys and result.get(k) is not None:
                result[k] = result[k] + v
            else:
                result[k] = v
    return result


def cell_cache_needs_update(cached: torch.Tensor | None, cell: torch.Tensor, rtol: float = 1e-5,
                            atol: float | None = None) -> bool:
    if cached is None or cached.shape != cell.shape or cached.device != cell.device:
        return True
    return not torch.allclose(cached, cell, rtol=rtol, atol=atol if atol is not None else 1e-8)
