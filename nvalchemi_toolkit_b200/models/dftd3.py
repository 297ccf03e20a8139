# SPDX-License-Identifier: Apache-2.0
"""DFT-D3 dispersion correction with Becke-Johnson damping.

Reference: ``nvalchemi/models/dftd3.py:115-431`` (parameter files) and ``:434-863`` (wrapper).  Two-body D3(BJ):
coordination numbers, Gaussian-interpolated ``C6(CN_i, CN_j)``, ``C8 = 3 C6 sqrt(Q_i Q_j)``,
``E = -1/2 sum_ij [s6 C6 / (r^6 + f^6) + s8 C8 / (r^8 + f^8)]``, ``f = a1 sqrt(C8/C6) + a2``, a smoothing window on the last
part of the cutoff, analytic forces (including the chain term through the coordination numbers), per-atom energies and
per-system virials.  The kernels work in atomic units; this wrapper converts from and to Angstrom / eV.

Parameters: the reference-C6 tables are data files (the reference downloads them); no network is assumed here.  Load
them with :meth:`DFTD3Parameters.load` (a ``.pt`` / ``.npz`` with ``rcov``, ``r4r2``, ``c6ref``, ``cnref``) or
:meth:`DFTD3Parameters.from_reference_table` (the flat five-column table of the original distribution);
:meth:`DFTD3Parameters.synthetic` makes smooth placeholder tables for tests and benchmarks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops

BOHR_A = 0.529177210903
HARTREE_EV = 27.211386245988
K1, K3, NREF = 16.0, 4.0, 5

#: Becke-Johnson damping parameters (s6, s8, a1, a2 [Bohr]) of common functionals (Grimme et al., J. Comput. Chem. 2011).
BJ_PARAMETERS: dict[str, tuple[float, float, float, float]] = {
    "pbe": (1.0, 0.7875, 0.4289, 4.4407), "pbe0": (1.0, 1.2177, 0.4145, 4.8593), "b3lyp": (1.0, 1.9889, 0.3981, 4.4211),
    "blyp": (1.0, 2.6996, 0.4298, 4.2359), "tpss": (1.0, 1.9435, 0.4535, 4.4752), "revpbe": (1.0, 2.3550, 0.5238, 3.5016),
    "hf": (1.0, 0.9171, 0.3385, 2.8830),
}


@dataclass
class DFTD3Parameters:
    """Element tables indexed by atomic number (row 0 unused): ``rcov [Z]`` (Bohr, already scaled by 4/3),
    ``r4r2 [Z]`` (``sqrt(Q)``), ``c6ref [Z,Z,5,5]`` (Hartree Bohr^6, ``<= 0`` marks an unused reference pair),
    ``cnref [Z,5]``."""

    rcov: torch.Tensor
    r4r2: torch.Tensor
    c6ref: torch.Tensor
    cnref: torch.Tensor

    def to(self, device: Any) -> "DFTD3Parameters":
        return DFTD3Parameters(*(t.to(device=device, dtype=torch.float64).contiguous()
                                 for t in (self.rcov, self.r4r2, self.c6ref, self.cnref)))

    def save(self, path: str | Path) -> None:
        torch.save({"rcov": self.rcov, "r4r2": self.r4r2, "c6ref": self.c6ref, "cnref": self.cnref}, Path(path))

    @classmethod
    def load(cls, path: str | Path) -> "DFTD3Parameters":
        path = Path(path)
        if path.suffix == ".npz":
            import numpy as np

            z = np.load(path)
            return cls(*(torch.from_numpy(z[k]).double() for k in ("rcov", "r4r2", "c6ref", "cnref")))
        d = torch.load(path, map_location="cpu", weights_only=True)
        return cls(d["rcov"].double(), d["r4r2"].double(), d["c6ref"].double(), d["cnref"].double())

    @classmethod
    def from_reference_table(cls, table: torch.Tensor, rcov: torch.Tensor, r4r2: torch.Tensor, max_z: int = 94
                             ) -> "DFTD3Parameters":
        """Build from the flat ``[n, 5]`` table ``(C6, Z_i + 100 a, Z_j + 100 b, CN_i, CN_j)`` where ``a, b`` are the
        reference indices (0..4) folded into the element codes."""
        c6 = torch.full((max_z + 1, max_z + 1, NREF, NREF), -1.0, dtype=torch.float64)
        cn = torch.full((max_z + 1, NREF), -1.0, dtype=torch.float64)
        for val, ci, cj, cni, cnj in table.double().tolist():
            zi, a = int(ci) % 100, int(ci) // 100
            zj, b = int(cj) % 100, int(cj) // 100
            if zi > max_z or zj > max_z:
                continue
            c6[zi, zj, a, b] = val
            c6[zj, zi, b, a] = val
            cn[zi, a], cn[zj, b] = cni, cnj
        return cls(rcov.double(), r4r2.double(), c6, cn)

    @classmethod
    def synthetic(cls, max_z: int = 94, seed: int = 0) -> "DFTD3Parameters":
        """Smooth, physically shaped placeholder tables (NOT the published parameters)."""
        g = torch.Generator().manual_seed(seed)
        z = torch.arange(max_z + 1, dtype=torch.float64)
        rcov = (0.6 + 0.35 * z.clamp_min(1) ** (1.0 / 3.0)) * (4.0 / 3.0) / BOHR_A * 0.5
        r4r2 = 1.5 + 2.5 * z.clamp_min(1) ** (1.0 / 3.0) / 2.0
        cnref = torch.stack([torch.linspace(0.0, 1.0, NREF, dtype=torch.float64) * (1.0 + (zz % 7)) for zz in range(max_z + 1)])
        base = 5.0 + 3.0 * z.clamp_min(1) ** 1.3
        amp = torch.sqrt(base[:, None] * base[None, :])
        damp = 1.0 / (1.0 + 0.15 * (torch.arange(NREF)[:, None] + torch.arange(NREF)[None, :]).double())
        jitter = 1.0 + 0.05 * torch.rand(max_z + 1, max_z + 1, NREF, NREF, generator=g, dtype=torch.float64)
        c6 = amp[:, :, None, None] * damp[None, None] * jitter
        c6 = 0.5 * (c6 + c6.permute(1, 0, 3, 2))
        c6[:, :, NREF - 1, :] = -1.0  # leave one reference unused, as real tables do for light elements
        c6[:, :, :, NREF - 1] = -1.0
        return cls(rcov, r4r2, c6, cnref)


def _pairs(pos, cells, nm, shifts, num, batch_idx):
    n, k = nm.shape
    valid = torch.arange(k, device=nm.device)[None] < num[:, None].clamp_max(k)
    i = torch.arange(n, device=nm.device)[:, None].expand(n, k)[valid]
    j = nm[valid].long()
    ok = j < n
    i, j, sh = i[ok], j[ok], shifts[valid][ok]
    d = pos[j] + torch.einsum("ei,eij->ej", sh.to(pos.dtype), cells[batch_idx.long()[i]]) - pos[i]
    return i, j, d


def d3_energy_torch(pos, cells, nm, shifts, num, batch_idx, z, p: DFTD3Parameters, s6, s8, a1, a2, r_on, cutoff,
                    cn_cutoff, weights=None) -> tuple[torch.Tensor, torch.Tensor]:
    """Differentiable per-atom energies (Hartree) and coordination numbers; positions and cells in Bohr."""
    n = pos.shape[0]
    i, j, d = _pairs(pos, cells, nm, shifts, num, batch_idx)
    r = d.norm(dim=-1)
    m_cn = r < cn_cutoff
    rc = p.rcov[z[i]] + p.rcov[z[j]]
    count = torch.where(m_cn, 1.0 / (1.0 + torch.exp(-K1 * (rc / r - 1.0))), torch.zeros_like(r))
    cn = torch.zeros(n, dtype=pos.dtype, device=pos.device).index_add_(0, i, count)
    ref = p.c6ref[z[i], z[j]]                                  # [E,5,5]
    di = cn[i][:, None] - p.cnref[z[i]]                        # [E,5]
    dj = cn[j][:, None] - p.cnref[z[j]]
    dist = di[:, :, None] ** 2 + dj[:, None, :] ** 2
    used = ref > 0
    dmin = torch.where(used, dist, torch.full_like(dist, float("inf"))).amin(dim=(1, 2), keepdim=True).detach()
    lw = torch.where(used, torch.exp(-K3 * (dist - dmin)), torch.zeros_like(dist))
    c6 = (lw * ref.clamp_min(0)).sum((1, 2)) / lw.sum((1, 2)).clamp_min(1e-300)
    qq = 3.0 * p.r4r2[z[i]] * p.r4r2[z[j]]
    f = a1 * torch.sqrt(qq) + a2
    e = -c6 * (s6 / (r ** 6 + f ** 6) + s8 * qq / (r ** 8 + f ** 8))
    x = ((r - r_on) / (cutoff - r_on)).clamp(0, 1)
    e = e * (1.0 - x ** 3 * (10.0 - 15.0 * x + 6.0 * x * x))
    e = torch.where(r < cutoff, e, torch.zeros_like(e))
    e_atom = torch.zeros(n, dtype=pos.dtype, device=pos.device).index_add_(0, i, 0.5 * e)
    return e_atom, cn


class DFTD3ModelWrapper(nn.Module, BaseModelMixin):
    def __init__(self, functional: str | None = "pbe", parameters: DFTD3Parameters | str | Path | None = None,
                 cutoff: float = 15.0, cn_cutoff: float | None = None, smoothing_width: float = 1.0,
                 s6: float | None = None, s8: float | None = None, a1: float | None = None, a2: float | None = None) -> None:
        super().__init__()
        base = BJ_PARAMETERS[functional.lower()] if functional is not None else (1.0, 0.0, 0.0, 0.0)
        self.s6, self.s8, self.a1, self.a2 = (v if v is not None else b for v, b in zip((s6, s8, a1, a2), base))
        self.functional = functional
        if parameters is None:
            raise ValueError("DFT-D3 needs its reference tables: pass parameters=DFTD3Parameters.load(path) "
                             "(or DFTD3Parameters.synthetic() for tests)")
        self.params = parameters if isinstance(parameters, DFTD3Parameters) else DFTD3Parameters.load(parameters)
        self.cutoff = float(cutoff)
        self.cn_cutoff = float(cn_cutoff) if cn_cutoff is not None else min(self.cutoff, 21.0 * BOHR_A)
        self.smoothing_width = float(smoothing_width)
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress", "virial", "atomic_energies", "coordination_numbers"}),
            optional_inputs=frozenset({"cell", "pbc", "neighbor_matrix_shifts"}), supports_pbc=True,
            neighbor_config=NeighborConfig(cutoff=self.cutoff, format=NeighborListFormat.MATRIX, half_list=False),
            active_outputs={"energy", "forces"})
        self._dev_params: tuple[Any, DFTD3Parameters] | None = None

    def _p(self, device: torch.device) -> DFTD3Parameters:
        if self._dev_params is None or self._dev_params[0] != device:
            self._dev_params = (device, self.params.to(device))
        return self._dev_params[1]

    def forward(self, data: Any, **kwargs: Any) -> dict:
        pos = data.positions
        n, dev, dtype = pos.shape[0], pos.device, pos.dtype
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        batch_idx = data.batch_idx if hasattr(data, "batch_idx") else torch.zeros(n, dtype=torch.int32, device=dev)
        cell = getattr(data, "cell", None)
        cells = cell.reshape(nb, 3, 3) if cell is not None else torch.eye(3, device=dev, dtype=dtype).expand(nb, 3, 3)
        nm, num = data.neighbor_matrix, data.num_neighbors
        sh = getattr(data, "neighbor_matrix_shifts", None)
        if sh is None:
            sh = torch.zeros(nm.shape + (3,), dtype=torch.int32, device=dev)
        weights = getattr(data, "energy_weights", None)
        p = self._p(dev)
        z = data.atomic_numbers.long()
        cut, cn_cut = self.cutoff / BOHR_A, self.cn_cutoff / BOHR_A
        r_on = (self.cutoff - self.smoothing_width) / BOHR_A
        if _native.require(pos):
            pb = (pos.detach().double() / BOHR_A).contiguous()
            cb = (cells.detach().double() / BOHR_A).contiguous()
            b32 = batch_idx.to(torch.int32).contiguous()
            nmc, shc, numc = nm.contiguous(), sh.contiguous(), num.contiguous()
            cn = _nops.d3_coordination(pb, cb, nmc, shc, numc, b32, z, p.rcov, cn_cut)
            prm = torch.tensor([self.s6, self.s8, self.a1, self.a2, r_on, cut], dtype=torch.float64)
            w64 = None if weights is None else weights.double().contiguous()
            e_atom, forces, virial, dcn = _nops.d3_pair(pb, cb, nmc, shc, numc, b32, z, cn, p.c6ref, p.cnref, p.r4r2, prm,
                                                        w64, nb)
            _nops.d3_cn_forces(pb, cb, nmc, shc, numc, b32, z, p.rcov, dcn, cn_cut, forces, virial)
            virial = virial.reshape(nb, 3, 3)
        else:
            with torch.enable_grad():
                pb = (pos.detach().double() / BOHR_A).requires_grad_(True)
                strain = torch.zeros(nb, 3, 3, dtype=torch.float64, device=dev, requires_grad=True)
                deform = torch.eye(3, dtype=torch.float64, device=dev) + 0.5 * (strain + strain.transpose(1, 2))
                ps = torch.einsum("ni,nij->nj", pb, deform[batch_idx.long()])
                cs = (cells.detach().double() / BOHR_A) @ deform
                e_atom, cn = d3_energy_torch(ps, cs, nm, sh, num, batch_idx, z, p, self.s6, self.s8, self.a1, self.a2,
                                             r_on, cut, cn_cut)
                total = (e_atom if weights is None else e_atom * weights.double()).sum()
                gp, gs = torch.autograd.grad(total, [pb, strain])
            forces, virial, e_atom = -gp, -gs, e_atom.detach()
        e_atom = e_atom * HARTREE_EV
        e_sum = e_atom if weights is None else e_atom * weights.double()
        energy = torch.zeros(nb, dtype=torch.float64, device=dev).index_add_(0, batch_idx.long(), e_sum)
        virial = virial * HARTREE_EV
        vol = torch.linalg.det(cells.detach().double()).abs().clamp_min(1e-30)
        out = {"energy": energy.to(dtype).unsqueeze(-1), "forces": (forces * (HARTREE_EV / BOHR_A)).to(dtype),
               "virial": virial.to(dtype), "stress": (-virial / vol[:, None, None]).to(dtype),
               "atomic_energies": e_atom.to(dtype), "coordination_numbers": cn.detach().to(dtype)}
        return self.adapt_output(out, data)

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed.spec import SPEC_DFTD3_HALO

        return SPEC_DFTD3_HALO
