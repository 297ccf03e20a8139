# SPDX-License-Identifier: Apache-2.0
"""One-shot neighbour construction on a ``Batch`` (reference ``nvalchemi/neighbors.py:55-277``).

``compute_neighbors`` builds the dense neighbour matrix with the cell-list kernel
(``_nops.neighbor_matrix_build``; CUDA and CPU), retries with a 1.5x wider matrix on overflow,
and stores either the MATRIX keys on the atoms group or a COO ``neighbor_list [E,2]`` + integer
``neighbor_list_shifts`` as a new edges group.  An edge ``(i, j, S)`` means: the image of ``j`` at
``r_j + S @ cell`` is within the cutoff of ``i``.
"""
from __future__ import annotations

import math

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.level_storage import SegmentedLevelStorage
from nvalchemi_toolkit_b200.models.base import NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


def estimate_max_neighbors(cutoff: float, density: float = 0.2, safety: float = 1.0) -> int:
    """Matrix width from a number density (atoms / A^3), rounded up to a multiple of 16."""
    k = 4.0 / 3.0 * math.pi * cutoff ** 3 * density * safety
    return max(16, int(math.ceil(k / 16.0)) * 16)


def cell_and_pbc(batch: Batch) -> tuple[torch.Tensor, torch.Tensor]:
    """``cell [B,3,3]`` and ``pbc [B,3]`` with identity / False defaults for non-periodic batches."""
    b, dev, dtype = batch.num_graphs, batch.device, batch.positions.dtype
    cell = getattr(batch, "cell", None)
    pbc = getattr(batch, "pbc", None)
    if cell is None:
        cell = torch.eye(3, dtype=dtype, device=dev).expand(b, 3, 3).contiguous()
    if pbc is None:
        pbc = torch.zeros(b, 3, dtype=torch.bool, device=dev)
    cell = cell.reshape(b, 3, 3)
    # non-periodic systems may carry a zero cell: use identity so fractional coordinates are defined
    # (explicit 3 x 3 determinant and an unconditional select: no library call, no host synchronisation per step)
    c = cell.double()
    det = (c[:, 0, 0] * (c[:, 1, 1] * c[:, 2, 2] - c[:, 1, 2] * c[:, 2, 1])
           - c[:, 0, 1] * (c[:, 1, 0] * c[:, 2, 2] - c[:, 1, 2] * c[:, 2, 0])
           + c[:, 0, 2] * (c[:, 1, 0] * c[:, 2, 1] - c[:, 1, 1] * c[:, 2, 0]))
    degenerate = det.abs() < 1e-12
    cell = torch.where(degenerate[:, None, None], torch.eye(3, dtype=cell.dtype, device=dev), cell)
    return cell.contiguous(), pbc.reshape(b, 3).to(torch.bool).contiguous()


def neighbor_matrix(positions: torch.Tensor, cell: torch.Tensor, pbc: torch.Tensor, batch_idx: torch.Tensor,
                    batch_ptr: torch.Tensor, cutoff: float, max_neighbors: int, half_list: bool = False,
                    out: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                    rebuild_flags: torch.Tensor | None = None, num_rows: int | None = None,
                    ghost_pull: tuple[int, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor] | None = None
                    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Dense neighbour search.  Returns ``(matrix [N,K] int32 padded with N, counts [N] int32, shifts [N,K,3] int32)``.

    With ``num_rows`` only the first ``num_rows`` atoms get a neighbour row (all atoms remain candidates): under domain
    decomposition ghost atoms send but do not receive, so their rows are never read.  ``ghost_pull = (first ghost row,
    home_rank, home_row, shift [G, 3], src_ptrs)`` (peer-memory decomposition, float32 CUDA): the first pass over the atoms
    fetches the ghost rows of ``positions`` from their owners and stores them IN ``positions`` before binning."""
    n = positions.shape[0]
    dev = positions.device
    if out is None:
        nm = torch.full((n, max_neighbors), n, dtype=torch.int32, device=dev)
        num = torch.zeros(n, dtype=torch.int32, device=dev)
        sh = torch.zeros(n, max_neighbors, 3, dtype=torch.int32, device=dev)
    else:
        nm, num, sh = out
    if n == 0:
        return nm, num, sh
    if _native.require(positions):
        if ghost_pull is not None and not (positions.is_contiguous() and positions.dtype == torch.float32):
            raise ValueError("ghost_pull writes the ghost rows into `positions`: pass a contiguous float32 tensor")
        _nops.neighbor_matrix_build(positions.detach().contiguous(), cell, pbc, batch_idx.to(torch.int32),
                                                  batch_ptr.to(torch.int32), float(cutoff), bool(half_list), nm, num, sh,
                                                  rebuild_flags, -1 if num_rows is None else int(num_rows),
                                                  *((None, None, None, None, -1) if ghost_pull is None else
                                                    (ghost_pull[1], ghost_pull[2], ghost_pull[3], ghost_pull[4], int(ghost_pull[0]))))
        return nm, num, sh
    if ghost_pull is not None:
        raise RuntimeError("ghost_pull needs the native library and CUDA positions")
    if num_rows is not None and num_rows < n:
        full = _neighbor_matrix_torch(positions.detach(), cell, pbc, batch_idx, cutoff, torch.full((n, nm.shape[1]), n, dtype=torch.int32, device=dev),
                                      torch.zeros(n, dtype=torch.int32, device=dev),
                                      torch.zeros(n, nm.shape[1], 3, dtype=torch.int32, device=dev), half_list)
        nm[:num_rows], num[:num_rows], sh[:num_rows] = full[0][:num_rows], full[1][:num_rows], full[2][:num_rows]
        return nm, num, sh
    return _neighbor_matrix_torch(positions.detach(), cell, pbc, batch_idx, cutoff, nm, num, sh, half_list)


def _neighbor_matrix_torch(pos, cell, pbc, batch_idx, cutoff, nm, num, sh, half_list):
    """Brute-force fallback (library not built): O(N^2 * images) per system, for small CPU cases only."""
    n, k = nm.shape
    nm.fill_(n)
    num.zero_()
    sh.zero_()
    b = batch_idx.long()
    for s in range(cell.shape[0]):
        idx = torch.nonzero(b == s).squeeze(1)
        if idx.numel() == 0:
            continue
        H = cell[s].double()
        inv = torch.linalg.inv(H)
        face = 1.0 / inv.norm(dim=0)
        reps = [int(math.ceil(cutoff / float(face[d]))) if bool(pbc[s, d]) else 0 for d in range(3)]
        rng = [torch.arange(-r, r + 1) for r in reps]
        S = torch.cartesian_prod(*rng).reshape(-1, 3).to(pos.device)
        p = pos[idx].double()
        frac = p @ inv
        w = torch.where(pbc[s], torch.floor(frac), torch.zeros_like(frac))
        pw = p - w @ H
        d = pw[None, :, None, :] + (S.double() @ H)[None, None, :, :] - pw[:, None, None, :]  # [i, j, S, 3]
        ok = (d * d).sum(-1) < cutoff * cutoff
        ii, jj, ss = torch.nonzero(ok, as_tuple=True)
        keep = ~((ii == jj) & (S[ss] == 0).all(-1))
        ii, jj, ss = ii[keep], jj[keep], ss[keep]
        Stot = S[ss] - w[jj].long() + w[ii].long()
        if half_list:
            gt = (jj > ii) | ((jj == ii) & ((Stot[:, 0] > 0) | ((Stot[:, 0] == 0) & ((Stot[:, 1] > 0) | ((Stot[:, 1] == 0) & (Stot[:, 2] > 0))))))
            ii, jj, Stot = ii[gt], jj[gt], Stot[gt]
        order = torch.argsort(ii, stable=True)
        ii, jj, Stot = ii[order], jj[order], Stot[order]
        cnt = torch.bincount(ii, minlength=idx.numel())
        start = torch.cumsum(cnt, 0) - cnt
        slot = torch.arange(ii.numel(), device=pos.device) - start[ii]
        fits = slot < k
        nm[idx[ii[fits]], slot[fits]] = idx[jj[fits]].to(torch.int32)
        sh[idx[ii[fits]], slot[fits]] = Stot[fits].to(torch.int32)
        num[idx] = cnt.to(torch.int32)
    return nm, num, sh


def neighbor_matrix_to_coo(nm: torch.Tensor, num: torch.Tensor, shifts: torch.Tensor | None
                           ) -> tuple[torch.Tensor, torch.Tensor | None]:
    """``(neighbor_list [E,2] int64 = (i, j), neighbor_list_shifts [E,3] int32)`` in row-major order."""
    n, k = nm.shape
    valid = torch.arange(k, device=nm.device)[None, :] < num[:, None].clamp_max(k)
    src = torch.arange(n, device=nm.device)[:, None].expand(n, k)[valid]
    nl = torch.stack([src, nm[valid].long()], dim=1)
    return nl, (shifts[valid] if shifts is not None else None)


def write_neighbor_data_to_batch(batch: Batch, nm: torch.Tensor, num: torch.Tensor, shifts: torch.Tensor | None,
                                 format: NeighborListFormat, cutoff: float) -> None:
    if format == NeighborListFormat.COO:
        nl, nls = neighbor_matrix_to_coo(nm, num, shifts)
        per_graph = torch.bincount(batch.batch_idx.long()[nl[:, 0]], minlength=batch.num_graphs).to(torch.int32)
        data = {"neighbor_list": nl}
        if nls is not None:
            data["neighbor_list_shifts"] = nls
            cell, _ = cell_and_pbc(batch)
            data["shifts"] = torch.einsum("ei,eij->ej", nls.to(cell.dtype), cell[batch.batch_idx.long()[nl[:, 0]]])
        batch._storage.groups["edges"] = SegmentedLevelStorage(data, per_graph, num_elements=int(nl.shape[0]),
                                                               device=batch.device)
    else:
        g = batch._atoms_group
        for key, val in (("neighbor_matrix", nm), ("num_neighbors", num), ("neighbor_matrix_shifts", shifts)):
            if val is None:
                continue
            if key in g.data and g.data[key].shape != val.shape:
                del g.data[key]
            g[key] = val
    object.__setattr__(batch, "_neighbor_list_cutoff", cutoff)


def compute_neighbors(batch: Batch, cutoff: float | None = None, *, config: NeighborConfig | None = None,
                      format: NeighborListFormat = NeighborListFormat.MATRIX, max_neighbors: int | None = None,
                      half_list: bool = False) -> None:
    if config is not None:
        cutoff, format, half_list = config.cutoff, config.format, config.half_list
    elif cutoff is None:
        raise ValueError("Either 'cutoff' or 'config' must be provided.")
    cell, pbc = cell_and_pbc(batch)
    if max_neighbors is None:
        max_neighbors = estimate_max_neighbors(cutoff)
        if not bool(pbc.any()) and batch.max_num_nodes > 0:
            max_neighbors = min(max_neighbors, (batch.max_num_nodes + 15) // 16 * 16)
    while True:
        nm, num, sh = neighbor_matrix(batch.positions, cell, pbc, batch.batch_idx, batch.batch_ptr, cutoff,
                                      max_neighbors, half_list)
        actual = int(num.max()) if num.numel() else 0
        if actual <= max_neighbors:
            break
        max_neighbors = ((int(actual * 1.5) + 1) + 15) // 16 * 16
    write_neighbor_data_to_batch(batch, nm, num, sh, format, cutoff)
