# SPDX-License-Identifier: Apache-2.0
"""Shared machinery of the Ewald and particle-mesh Ewald models.

Physics (reference ``nvalchemi/models/_ops/electrostatics/ewald.py:78-923``, ``pme.py:94-788``, ``slab.py:83-450``):
``E = E_real + E_recip + E_self + E_background (+ E_slab)`` with splitting parameter ``alpha``,

* ``E_real  = 1/2 sum_{i != j} q_i q_j erfc(alpha r_ij) / r_ij`` over the neighbour list,
* ``E_recip = (2 pi / V) sum_{k != 0} exp(-k^2 / 4 alpha^2) / k^2 |S(k)|^2``, ``S(k) = sum_i q_i exp(i k.r_i)``
  (summed directly over a half space of k-vectors, or on a B-spline mesh),
* ``E_self = -alpha / sqrt(pi) sum_i q_i^2``, ``E_background = -pi Q^2 / (2 V alpha^2)``,
* ``E_slab = (2 pi / V) M_z^2`` for systems periodic in x, y only.

All pieces come with analytic forces, virials ``W = -dE/d(strain)`` and potentials ``phi_i = dE/dq_i``; the autograd
function at the end exposes them as gradients, so a charge-predicting model upstream can be trained through the energy.
Energies are multiplied by the Coulomb constant ``e^2 / (4 pi eps0) = 14.3996 eV A``.
"""
from __future__ import annotations

import math
from typing import Any

import torch

from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops

COULOMB_EV_A = 14.399645478425668


def estimate_ewald_parameters(cutoff: float, accuracy: float = 1e-6) -> tuple[float, float]:
    """``(alpha, k_cutoff)`` for a real-space cutoff and a relative accuracy (both truncation errors ~ accuracy)."""
    t = math.sqrt(-math.log(accuracy))
    alpha = t / cutoff
    return alpha, 2.0 * alpha * t


def generate_k_vectors(cell: torch.Tensor, k_cutoff: float) -> torch.Tensor:
    """Half-space reciprocal vectors ``k = 2 pi inv(cell) m`` with ``0 < |k| <= k_cutoff`` (float64 ``[K,3]``)."""
    cell = cell.detach().double().reshape(3, 3).cpu()
    recip = 2.0 * math.pi * torch.linalg.inv(cell)  # columns are reciprocal vectors
    lim = [int(math.floor(k_cutoff * float(cell[d].norm()) / (2.0 * math.pi))) + 1 for d in range(3)]
    rng = [torch.arange(-l, l + 1, dtype=torch.float64) for l in lim]
    m = torch.stack(torch.meshgrid(*rng, indexing="ij"), -1).reshape(-1, 3)
    half = (m[:, 0] > 0) | ((m[:, 0] == 0) & (m[:, 1] > 0)) | ((m[:, 0] == 0) & (m[:, 1] == 0) & (m[:, 2] > 0))
    m = m[half]
    k = m @ recip.t()
    return k[k.norm(dim=-1) <= k_cutoff].contiguous()


def _good_fft_size(n: int) -> int:
    while True:
        m = n
        for p in (2, 3, 5, 7):
            while m % p == 0:
                m //= p
        if m == 1:
            return n
        n += 1


def pme_mesh_dims(cell: torch.Tensor, alpha: float, accuracy: float = 1e-6, spacing: float | None = None,
                  order: int = 5) -> tuple[int, int, int]:
    """Mesh points per cell vector: spacing ``h`` chosen so that the aliasing error of the order-``p`` spline at the
    reciprocal cutoff stays near ``accuracy`` (``h ~ (accuracy)^(1/p) / alpha`` scaled), rounded to FFT-friendly sizes."""
    cell = cell.detach().double().reshape(3, 3).cpu()
    if spacing is None:
        spacing = min(1.0, 1.5 * accuracy ** (1.0 / (2.0 * order)) / alpha * 1.0)
    return tuple(_good_fft_size(max(order + 1, int(math.ceil(float(cell[d].norm()) / spacing)))) for d in range(3))


def bspline_moduli(n: int, order: int) -> torch.Tensor:
    """``|b(m)|^2`` of the Euler exponential spline for a mesh of ``n`` points (float64 ``[n]``)."""
    # M_p at the integer knots 1..p-1 by the recursion on a fine evaluation of the cardinal spline
    m = torch.zeros(order + 1, dtype=torch.float64)
    m[1] = 1.0  # M_2 at integer knots 0,1,2: (0, 1, 0)
    for p in range(3, order + 1):
        new = torch.zeros_like(m)
        for k in range(1, p):
            new[k] = (k * m[k] + (p - k) * m[k - 1]) / (p - 1)
        m = new
    knots = m[1:order]  # M_p(1..p-1)
    idx = torch.arange(n, dtype=torch.float64)
    ks = torch.arange(order - 1, dtype=torch.float64)
    ph = 2.0 * math.pi * idx[:, None] * ks[None] / n
    den = (knots[None] * torch.cos(ph)).sum(-1) ** 2 + (knots[None] * torch.sin(ph)).sum(-1) ** 2
    small = den < 1e-10
    if small.any():  # even orders at the Nyquist index: average the neighbours (Essmann et al. 1995)
        den = den.clone()
        for i in torch.nonzero(small).flatten().tolist():
            den[i] = 0.5 * (den[(i - 1) % n] + den[(i + 1) % n])
    return 1.0 / den


# ---- pieces -----------------------------------------------------------------------------------------------------
def real_space(positions, charges, cells, nm, shifts, num, batch_idx, alpha, cutoff, half_list, num_systems):
    """Per-atom energies, forces, virials ``[B,3,3]`` and potentials of the screened real-space sum."""
    if shifts is None:
        shifts = torch.zeros(nm.shape + (3,), dtype=torch.int32, device=nm.device)
    if _native.require(positions):
        e, f, w, phi = _nops.ewald_real(positions.detach().contiguous(), charges.detach().to(positions.dtype).contiguous(),
                                        cells.detach().to(positions.dtype).contiguous(), nm.contiguous(), shifts.contiguous(),
                                        num.contiguous(), batch_idx.to(torch.int32).contiguous(), alpha.double().contiguous(),
                                        int(positions.shape[0]), float(cutoff), bool(half_list), int(num_systems))
        return e, f, w.reshape(num_systems, 3, 3), phi
    return _real_space_torch(positions, charges, cells, nm, shifts, num, batch_idx, alpha, cutoff, half_list, num_systems)


def _real_space_torch(pos, q, cells, nm, shifts, num, batch_idx, alpha, cutoff, half, nsys):
    n, k = nm.shape
    valid = torch.arange(k, device=nm.device)[None] < num[:, None].clamp_max(k)
    i = torch.arange(n, device=nm.device)[:, None].expand(n, k)[valid]
    j = nm[valid].long()
    ok = j < n
    i, j, sh = i[ok], j[ok], shifts[valid][ok]
    b = batch_idx.long()
    p, qd = pos.detach().double(), q.detach().double()
    d = p[j] + torch.einsum("ei,eij->ej", sh.double(), cells.double()[b[i]]) - p[i]
    r = d.norm(dim=-1)
    keep = (r < cutoff) & (r > 0)
    i, j, d, r = i[keep], j[keep], d[keep], r[keep]
    a = alpha.double()[b[i]]
    ec = torch.erfc(a * r) / r
    dec = -(ec + a * (2.0 / math.sqrt(math.pi)) * torch.exp(-(a * r) ** 2)) / r
    wgt = 1.0 if half else 0.5
    e_atom = torch.zeros(n, dtype=torch.float64, device=pos.device).index_add_(0, i, wgt * qd[i] * qd[j] * ec)
    phi = torch.zeros(n, dtype=torch.float64, device=pos.device).index_add_(0, i, qd[j] * ec)
    g = (qd[i] * qd[j] * dec / r)[:, None] * d
    f = torch.zeros(n, 3, dtype=torch.float64, device=pos.device).index_add_(0, i, g)
    if half:
        f.index_add_(0, j, -g)
        phi.index_add_(0, j, qd[i] * ec)
    w = torch.zeros(nsys, 3, 3, dtype=torch.float64, device=pos.device).index_add_(
        0, b[i], -wgt * d[:, :, None] * g[:, None, :])
    return e_atom.to(pos.dtype), f.to(pos.dtype), w.to(pos.dtype), phi.to(pos.dtype)


def structure_factors(positions, charges, kvecs, a0, a1, weights=None):
    if _native.require(positions):
        w = None if weights is None else weights.to(positions.dtype).contiguous()
        return _nops.ewald_structure_factors(positions.detach().contiguous(),
                                             charges.detach().to(positions.dtype).contiguous(), kvecs, int(a0), int(a1), w)
    q = charges.detach().double()[a0:a1]
    if weights is not None:
        q = q * weights.double()[a0:a1]
    ph = positions.detach().double()[a0:a1] @ kvecs.t()
    return torch.stack([(q[:, None] * torch.cos(ph)).sum(0), (q[:, None] * torch.sin(ph)).sum(0)], -1)


def recip_apply(positions, charges, kvecs, coef, sk, a0, a1):
    if _native.require(positions):
        return _nops.ewald_recip_apply(positions.detach().contiguous(), charges.detach().to(positions.dtype).contiguous(),
                                       kvecs, coef.contiguous(), sk.contiguous(), int(a0), int(a1))
    p = positions.detach().double()[a0:a1]
    q = charges.detach().double()[a0:a1]
    ph = p @ kvecs.t()
    cs, sn = torch.cos(ph), torch.sin(ph)
    im = sn * sk[:, 0] - cs * sk[:, 1]
    re = cs * sk[:, 0] + sn * sk[:, 1]
    f = q[:, None] * ((coef * im) @ kvecs)
    return f, (re * coef).sum(-1)


def recip_direct(positions, charges, cell, kvecs, alpha, a0, a1, weights=None, reduce=None):
    """Direct k-space sum for one system (atoms ``[a0,a1)``): energy, forces, virial ``[3,3]``, potentials."""
    vol = float(torch.linalg.det(cell.detach().double()).abs())
    k2 = (kvecs * kvecs).sum(-1)
    amp = torch.exp(-k2 / (4.0 * alpha * alpha)) / k2
    sk = structure_factors(positions, charges, kvecs, a0, a1, weights)
    if reduce is not None:
        sk = reduce(sk)
    s2 = (sk * sk).sum(-1)
    e_k = (4.0 * math.pi / vol) * amp * s2  # half-space terms carry twice the full-space weight
    energy = e_k.sum()
    vf = 2.0 * (1.0 / k2 + 1.0 / (4.0 * alpha * alpha))
    virial = torch.eye(3, dtype=torch.float64, device=kvecs.device) * energy - torch.einsum("k,ki,kj->ij", e_k * vf, kvecs, kvecs)
    f, phi = recip_apply(positions, charges, kvecs, (8.0 * math.pi / vol) * amp, sk, a0, a1)
    return energy, f, virial, phi


def recip_mesh(positions, charges, cell, alpha, dims, order, moduli, a0, a1, weights=None, reduce=None):
    """Particle-mesh reciprocal sum for one system: energy, forces, virial ``[3,3]``, potentials."""
    cell64 = cell.detach().double().reshape(3, 3)
    inv = torch.linalg.inv(cell64).contiguous()
    vol = float(torch.linalg.det(cell64).abs())
    nx, ny, nz = dims
    native = _native.require(positions)
    if native:
        w = None if weights is None else weights.to(positions.dtype).contiguous()
        mesh = _nops.pme_spread(positions.detach().contiguous(), charges.detach().to(positions.dtype).contiguous(), inv,
                                nx, ny, nz, int(order), int(a0), int(a1), w)
    else:
        mesh = _spread_torch(positions, charges, inv, dims, order, a0, a1, weights)
    if reduce is not None:
        mesh = reduce(mesh)
    fk = torch.fft.rfftn(mesh)
    if native:
        fk_real = torch.view_as_real(fk).contiguous()
        acc = _nops.pme_convolve(fk_real, inv, moduli[0], moduli[1], moduli[2], float(alpha), vol, nz)
        fk = torch.view_as_complex(fk_real)
        energy = acc[0]
        virial = torch.stack([acc[1], acc[2], acc[3], acc[2], acc[4], acc[5], acc[3], acc[5], acc[6]]).reshape(3, 3)
    else:
        fk, energy, virial = _convolve_torch(fk, inv, moduli, alpha, vol, dims)
    phi_mesh = torch.fft.irfftn(fk, s=(nx, ny, nz), norm="forward").contiguous()
    if native:
        f, phi = _nops.pme_gather(positions.detach().contiguous(), charges.detach().to(positions.dtype).contiguous(), inv,
                                  phi_mesh, int(order), int(a0), int(a1))
    else:
        f, phi = _gather_torch(positions, charges, inv, phi_mesh, dims, order, a0, a1)
    return energy, f, virial, phi


# ---- plain PyTorch mesh stages (oracle and CPU fallback) -----------------------------------------------------------
def _raise_order(v: torch.Tensor, w: torch.Tensor, k: int) -> torch.Tensor:
    """Spline values of order ``k`` from those of order ``k-1`` (slot ``s`` holds ``M(w + k - 1 - s)``)."""
    div = 1.0 / (k - 1)
    new = v.clone()
    new[:, k - 1] = div * w * v[:, k - 2]
    for j in range(1, k - 1):
        new[:, k - j - 1] = div * ((w + j) * v[:, k - j - 2] + (k - j - w) * v[:, k - j - 1])
    new[:, 0] = div * (1.0 - w) * v[:, 0]
    return new


def _spline_weights(w: torch.Tensor, order: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Cardinal B-spline values and derivatives on the ``order`` grid points below fractional offset ``w``."""
    v = torch.zeros(w.shape[0], order, dtype=torch.float64, device=w.device)
    v[:, 0], v[:, 1] = 1.0 - w, w
    for k in range(3, order):
        v = _raise_order(v, w, k)
    dv = torch.zeros_like(v)
    dv[:, 0] = -v[:, 0]
    dv[:, 1:] = v[:, :-1] - v[:, 1:]
    return _raise_order(v, w, order), dv


def _mesh_indices(positions, inv, dims, order, a0, a1):
    p = positions.detach().double()[a0:a1]
    frac = p @ inv
    frac = frac - torch.floor(frac)
    out = []
    for d in range(3):
        u = frac[:, d] * dims[d]
        fl = torch.floor(u)
        v, dv = _spline_weights(u - fl, order)
        idx = (fl.long()[:, None] - order + 1 + torch.arange(order, device=p.device)[None]) % dims[d]
        out.append((idx, v, dv))
    return out


def _spread_torch(positions, charges, inv, dims, order, a0, a1, weights):
    q = charges.detach().double()[a0:a1]
    if weights is not None:
        q = q * weights.double()[a0:a1]
    (ix, vx, _), (iy, vy, _), (iz, vz, _) = _mesh_indices(positions, inv, dims, order, a0, a1)
    w = q[:, None, None, None] * vx[:, :, None, None] * vy[:, None, :, None] * vz[:, None, None, :]
    flat = (ix[:, :, None, None] * dims[1] + iy[:, None, :, None]) * dims[2] + iz[:, None, None, :]
    mesh = torch.zeros(dims[0] * dims[1] * dims[2], dtype=torch.float64, device=q.device)
    mesh.index_add_(0, flat.reshape(-1), w.reshape(-1))
    return mesh.reshape(dims)


def _convolve_torch(fk, inv, moduli, alpha, vol, dims):
    nx, ny, nz = dims
    dev = fk.device
    mx = torch.fft.fftfreq(nx, 1.0 / nx, dtype=torch.float64, device=dev)
    my = torch.fft.fftfreq(ny, 1.0 / ny, dtype=torch.float64, device=dev)
    mz = torch.arange(nz // 2 + 1, dtype=torch.float64, device=dev)
    if nx % 2 == 0:
        mx[nx // 2] = nx // 2  # the kernels count the Nyquist index as positive
    if ny % 2 == 0:
        my[ny // 2] = ny // 2
    m = torch.stack(torch.meshgrid(mx, my, mz, indexing="ij"), -1)
    k = 2.0 * math.pi * m @ inv.t()
    k2 = (k * k).sum(-1)
    k2[0, 0, 0] = 1.0
    g = (4.0 * math.pi / vol) * torch.exp(-k2 / (4 * alpha * alpha)) / k2 * (
        moduli[0][:, None, None] * moduli[1][None, :, None] * moduli[2][None, None, : nz // 2 + 1])
    g[0, 0, 0] = 0.0
    wt = torch.full((nz // 2 + 1,), 2.0, dtype=torch.float64, device=dev)
    wt[0] = 1.0
    if nz % 2 == 0:
        wt[-1] = 1.0
    e = 0.5 * wt * g * (fk.real ** 2 + fk.imag ** 2)
    vf = 2.0 * (1.0 / k2 + 1.0 / (4 * alpha * alpha))
    energy = e.sum()
    virial = torch.eye(3, dtype=torch.float64, device=dev) * energy - torch.einsum("xyz,xyzi,xyzj->ij", e * vf, k, k)
    return fk * g, energy, virial


def _gather_torch(positions, charges, inv, phi_mesh, dims, order, a0, a1):
    q = charges.detach().double()[a0:a1]
    (ix, vx, dx), (iy, vy, dy), (iz, vz, dz) = _mesh_indices(positions, inv, dims, order, a0, a1)
    flat = (ix[:, :, None, None] * dims[1] + iy[:, None, :, None]) * dims[2] + iz[:, None, None, :]
    m = phi_mesh.double().reshape(-1)[flat]
    phi = (vx[:, :, None, None] * vy[:, None, :, None] * vz[:, None, None, :] * m).sum((1, 2, 3))
    g0 = (dx[:, :, None, None] * vy[:, None, :, None] * vz[:, None, None, :] * m).sum((1, 2, 3)) * dims[0]
    g1 = (vx[:, :, None, None] * dy[:, None, :, None] * vz[:, None, None, :] * m).sum((1, 2, 3)) * dims[1]
    g2 = (vx[:, :, None, None] * vy[:, None, :, None] * dz[:, None, None, :] * m).sum((1, 2, 3)) * dims[2]
    f = -q[:, None] * (torch.stack([g0, g1, g2], -1) @ inv.t())
    return f, phi
