# SPDX-License-Identifier: Apache-2.0
"""Integrator / thermostat / reduction operators (Python entry points).

Names and argument orders follow the reference's torch custom ops
(``nvalchemi/dynamics/_ops/*.py``, ``dynamics/hooks/_utils.py:58-170``,
``hooks/periodic.py:42-66``).  Every function mutates its first arguments in place exactly as the
reference op does.  With the native library loaded (always on a GPU machine) the work is done by
``torch.ops.nvalchemi.*`` kernels, which cover both CUDA and CPU tensors; without it (CPU-only
machine, library not built) an equivalent torch expression runs.

Time quantities are in internal units (``sqrt(amu A^2 / eV)``); temperatures passed to the
kernels are ``k_B T`` in eV.
"""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.dynamics._units import KB_EV
from nvalchemi_toolkit_b200.ops import _native
from nvalchemi_toolkit_b200.ops._native_counter import ops as _nops


def _nat(t: torch.Tensor) -> bool:
    return _native.require(t)


def _i32(b: torch.Tensor) -> torch.Tensor:
    return b if b.dtype == torch.int32 else b.to(torch.int32)


def _to_per_system(value: float | torch.Tensor, m: int, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Broadcast a scalar (or ``[M]`` tensor) to a contiguous ``[M]`` tensor."""
    if isinstance(value, torch.Tensor):
        return value.to(device=device, dtype=dtype).reshape(-1).expand(m).contiguous()
    return torch.full((m,), float(value), device=device, dtype=dtype)


# ------------------------------------------------------------------------ velocity Verlet
def vv_position_update(positions, velocities, forces, masses, dt, batch_idx) -> None:
    """``r += v dt + (F/2m) dt^2;  v += (F/2m) dt`` with per-system ``dt[M]``."""
    if _nat(positions):
        _nops.vv_position_update(positions, velocities, forces.contiguous(), masses, dt, _i32(batch_idx))
        return
    h = dt[batch_idx.long()].unsqueeze(-1)
    a = forces / masses.unsqueeze(-1)
    positions.add_(velocities * h + 0.5 * a * h * h)
    velocities.add_(0.5 * a * h)


def vv_velocity_finalize(velocities, forces_new, masses, dt, batch_idx) -> None:
    """``v += (F_new/2m) dt``."""
    if _nat(velocities):
        _nops.vv_velocity_finalize(velocities, forces_new.contiguous(), masses, dt, _i32(batch_idx))
        return
    h = dt[batch_idx.long()].unsqueeze(-1)
    velocities.add_(0.5 * h * forces_new / masses.unsqueeze(-1))


# ------------------------------------------------------------------------ Langevin (BAOAB)
def langevin_half_step(positions, velocities, forces, masses, dt, temperature, friction, random_seed, batch_idx,
                       atom_ids=None) -> None:
    """B-A-O-A part of BAOAB.  ``temperature`` is ``k_B T`` in eV per system; noise is a
    counter-based Philox stream keyed by ``(random_seed, atom index)`` so results do not depend on
    launch geometry (``atom_ids`` supplies global indices under domain decomposition)."""
    if _nat(positions):
        _nops.langevin_half_step(positions, velocities, forces.contiguous(), masses, dt, temperature,
                                               friction, int(random_seed), _i32(batch_idx), atom_ids)
        return
    b = batch_idx.long()
    h = dt[b].unsqueeze(-1)
    im = 1.0 / masses.unsqueeze(-1)
    gen = torch.Generator(device="cpu").manual_seed(int(random_seed))
    noise = torch.randn(positions.shape, generator=gen, dtype=torch.float64).to(positions)
    c1 = torch.exp(-friction[b] * dt[b]).unsqueeze(-1)
    c2 = torch.sqrt((1.0 - c1 * c1) * temperature[b].unsqueeze(-1) * im)
    velocities.add_(0.5 * h * forces * im)
    positions.add_(0.5 * h * velocities)
    velocities.mul_(c1).add_(c2 * noise)
    positions.add_(0.5 * h * velocities)


def langevin_finalize(velocities, forces_new, masses, dt, batch_idx) -> None:
    vv_velocity_finalize(velocities, forces_new, masses, dt, batch_idx)


# ------------------------------------------------------------------------ kinetic energy etc.
def compute_kinetic_energy(velocities, masses, batch_idx, num_systems: int) -> torch.Tensor:
    """Per-system ``sum_i m_i v_i^2 / 2`` → ``[M]`` (fp64 accumulation)."""
    if _nat(velocities):
        return _nops.compute_kinetic_energy(velocities.contiguous(), masses, _i32(batch_idx), num_systems)
    ke = 0.5 * masses.double() * (velocities.double() ** 2).sum(-1)
    out = torch.zeros(num_systems, dtype=torch.float64, device=velocities.device)
    return out.index_add_(0, batch_idx.long(), ke).to(velocities.dtype)


def compute_temperature(kinetic_energy: torch.Tensor, num_atoms_per_system: torch.Tensor) -> torch.Tensor:
    """``T = 2 KE / (3 N k_B)`` in kelvin."""
    return 2.0 * kinetic_energy / (3.0 * num_atoms_per_system.to(kinetic_energy.dtype).clamp_min(1) * KB_EV)


def momentum_sums(velocities, masses, batch_idx, num_systems: int) -> torch.Tensor:
    """``[M,4]`` fp64: ``(sum m v_x, sum m v_y, sum m v_z, sum m)``."""
    if _nat(velocities):
        return _nops.momentum_sums(velocities.contiguous(), masses, _i32(batch_idx), num_systems)
    mv = torch.cat([masses.double().unsqueeze(-1) * velocities.double(), masses.double().unsqueeze(-1)], dim=1)
    return torch.zeros(num_systems, 4, dtype=torch.float64, device=velocities.device).index_add_(0, batch_idx.long(), mv)


def _shift_scale(velocities, shift, scale, batch_idx) -> None:
    if _nat(velocities):
        _nops.velocity_shift_scale(velocities, shift.contiguous(), scale.contiguous(), _i32(batch_idx))
        return
    b = batch_idx.long()
    velocities.sub_(shift[b]).mul_(scale[b].unsqueeze(-1))


def remove_com_motion(velocities, masses, batch_idx, num_systems: int) -> None:
    s = momentum_sums(velocities, masses, batch_idx, num_systems)
    vcom = (s[:, :3] / s[:, 3:].clamp_min(1e-30)).to(velocities.dtype)
    _shift_scale(velocities, vcom, torch.ones(num_systems, dtype=velocities.dtype, device=velocities.device), batch_idx)


def velocity_rescale(velocities, scale_factor, batch_idx) -> None:
    m = scale_factor.shape[0]
    _shift_scale(velocities, torch.zeros(m, 3, dtype=velocities.dtype, device=velocities.device),
                 scale_factor.to(velocities.dtype), batch_idx)


def initialize_velocities(velocities, masses, temperature, batch_idx, random_seed: int = 42, remove_com: bool = True,
                          remove_rotations: bool = False, rescale: bool = True, positions=None, atom_ids=None) -> None:
    """Maxwell-Boltzmann draw at ``temperature`` (kelvin, scalar or ``[M]``), optional COM/rotation
    removal and exact rescale to the target temperature (3N degrees of freedom, as ``compute_temperature``)."""
    m = int(batch_idx.max().item()) + 1 if batch_idx.numel() else 0
    dev, dtype = velocities.device, velocities.dtype
    kT = _to_per_system(temperature, m, dev, dtype) * KB_EV
    b32 = _i32(batch_idx)
    if _nat(velocities):
        _nops.maxwell_boltzmann(velocities, masses, kT, b32, int(random_seed), atom_ids)
    else:
        gen = torch.Generator(device="cpu").manual_seed(int(random_seed))
        z = torch.randn(velocities.shape, generator=gen, dtype=torch.float64).to(velocities)
        velocities.copy_(z * torch.sqrt(kT[batch_idx.long()] / masses).unsqueeze(-1))
    if remove_com:
        remove_com_motion(velocities, masses, batch_idx, m)
    if remove_rotations and positions is not None:
        _remove_rotations(velocities, positions, masses, batch_idx, m)
    if rescale:
        ke = compute_kinetic_energy(velocities, masses, batch_idx, m)
        n_at = torch.bincount(batch_idx.long(), minlength=m)
        t_now = compute_temperature(ke, n_at)
        t_target = kT / KB_EV
        scale = torch.where(t_now > 0, torch.sqrt(t_target / t_now.clamp_min(1e-30)), torch.ones_like(t_now))
        velocity_rescale(velocities, scale, batch_idx)


def _remove_rotations(velocities, positions, masses, batch_idx, m: int) -> None:
    b = batch_idx.long()
    md = masses.double().unsqueeze(-1)
    msum = torch.zeros(m, 1, dtype=torch.float64, device=positions.device).index_add_(0, b, md)
    com = torch.zeros(m, 3, dtype=torch.float64, device=positions.device).index_add_(0, b, md * positions.double()) / msum
    r = positions.double() - com[b]
    L = torch.zeros(m, 3, dtype=torch.float64, device=positions.device).index_add_(
        0, b, md * torch.cross(r, velocities.double(), dim=-1))
    r2 = (r * r).sum(-1, keepdim=True)
    eye = torch.eye(3, dtype=torch.float64, device=positions.device)
    inertia_i = md.unsqueeze(-1) * (r2.unsqueeze(-1) * eye - r.unsqueeze(-1) * r.unsqueeze(-2))
    inertia = torch.zeros(m, 3, 3, dtype=torch.float64, device=positions.device).index_add_(0, b, inertia_i)
    omega = torch.linalg.solve(inertia + 1e-12 * eye, L.unsqueeze(-1)).squeeze(-1)
    velocities.sub_(torch.cross(omega[b], r, dim=-1).to(velocities.dtype))


# ------------------------------------------------------------------------ FIRE
def fire_step(positions, velocities, forces, masses, alpha, dt, n_steps_positive, alpha_start, f_alpha, dt_min, dt_max,
              maxstep, n_min, f_dec, f_inc, uphill_flag, *, vf=None, vv=None, ff=None, batch_idx=None,
              compute_reductions: bool = True, reduce_max=None) -> None:
    """One FIRE iteration (power test, velocity mixing, adaptive ``dt``/``alpha``, kick, capped drift).

    With ``compute_reductions=False`` the caller supplies ``vf, vv, ff`` already summed (for example
    across ranks of a domain decomposition), mirroring the reference seam
    (``nvalchemi/dynamics/_ops/fire.py:245-363``).  ``reduce_max`` (a callable ``Tensor -> Tensor``) is applied to the
    per-system largest displacement before the step-length cap, so that all ranks holding parts of one system scale
    their drift alike."""
    m = alpha.shape[0]
    dev, dtype = positions.device, positions.dtype
    if batch_idx is None:
        batch_idx = torch.zeros(positions.shape[0], dtype=torch.int32, device=dev)
    vf = vf if vf is not None else torch.zeros(m, dtype=dtype, device=dev)
    vv = vv if vv is not None else torch.zeros(m, dtype=dtype, device=dev)
    ff = ff if ff is not None else torch.zeros(m, dtype=dtype, device=dev)
    if _nat(positions):
        args = (positions, velocities, forces.contiguous(), masses, alpha, dt, alpha_start, f_alpha, dt_min, dt_max, maxstep,
                n_steps_positive, n_min, f_dec, f_inc, uphill_flag, vf, vv, ff, _i32(batch_idx), compute_reductions)
        if reduce_max is None:
            _nops._fire_step_op(*args)
        else:
            mx = torch.zeros(m, dtype=torch.float32, device=dev)
            _nops._fire_step_op(*args, mx, 1)
            mx.copy_(reduce_max(mx))
            _nops._fire_step_op(*args, mx, 2)
        return
    b = batch_idx.long()
    if compute_reductions:
        z = torch.zeros(m, dtype=torch.float64, device=dev)
        vf.copy_(z.clone().index_add_(0, b, (velocities.double() * forces.double()).sum(-1)))
        vv.copy_(z.clone().index_add_(0, b, (velocities.double() ** 2).sum(-1)))
        ff.copy_(z.clone().index_add_(0, b, (forces.double() ** 2).sum(-1)))
    pos_power = vf > 0
    n_steps_positive.copy_(torch.where(pos_power, n_steps_positive + 1, torch.zeros_like(n_steps_positive)))
    grow = pos_power & (n_steps_positive > n_min)
    keep = torch.where(pos_power, 1.0 - alpha, torch.zeros_like(alpha))
    mix = torch.where(pos_power & (ff > 0), alpha * torch.sqrt(vv / ff.clamp_min(1e-300)), torch.zeros_like(alpha))
    dt.copy_(torch.where(grow, torch.minimum(dt * f_inc, dt_max), torch.where(pos_power, dt, torch.maximum(dt * f_dec, dt_min))))
    alpha.copy_(torch.where(grow, alpha * f_alpha, torch.where(pos_power, alpha, alpha_start)))
    h = dt[b].unsqueeze(-1)
    velocities.mul_(keep[b].unsqueeze(-1)).add_(mix[b].unsqueeze(-1) * forces).add_(h * forces / masses.unsqueeze(-1))
    dr = h * velocities
    dn = dr.norm(dim=-1)
    mx = torch.zeros(m, dtype=dn.dtype, device=dev).scatter_reduce(0, b, dn, "amax", include_self=True)
    if reduce_max is not None:
        mx = reduce_max(mx)
    scale = torch.where(mx > maxstep, maxstep / mx.clamp_min(1e-30), torch.ones_like(mx))
    positions.add_(scale[b].unsqueeze(-1) * dr)


def fire_update(velocities, forces, alpha, dt, n_steps_positive, alpha_start, f_alpha, dt_min, dt_max, n_min, f_dec,
                f_inc, *, vf=None, vv=None, ff=None, batch_idx=None, compute_reductions: bool = True) -> None:
    """FIRE velocity mixing and controller update only (no kick, no drift); used by variable-cell FIRE."""
    m = alpha.shape[0]
    dev = velocities.device
    b = (batch_idx if batch_idx is not None else torch.zeros(velocities.shape[0], dtype=torch.int32, device=dev)).long()
    if compute_reductions or vf is None:
        z = torch.zeros(m, dtype=torch.float64, device=dev)
        rvf = z.clone().index_add_(0, b, (velocities.double() * forces.double()).sum(-1)).to(velocities.dtype)
        rvv = z.clone().index_add_(0, b, (velocities.double() ** 2).sum(-1)).to(velocities.dtype)
        rff = z.clone().index_add_(0, b, (forces.double() ** 2).sum(-1)).to(velocities.dtype)
        for dst, src in ((vf, rvf), (vv, rvv), (ff, rff)):
            if dst is not None:
                dst.copy_(src)
        vf, vv, ff = rvf, rvv, rff
    pos_power = vf > 0
    n_steps_positive.copy_(torch.where(pos_power, n_steps_positive + 1, torch.zeros_like(n_steps_positive)))
    grow = pos_power & (n_steps_positive > n_min)
    keep = torch.where(pos_power, 1.0 - alpha, torch.zeros_like(alpha))
    mix = torch.where(pos_power & (ff > 0), alpha * torch.sqrt(vv / ff.clamp_min(1e-300)), torch.zeros_like(alpha))
    dt.copy_(torch.where(grow, torch.minimum(dt * f_inc, dt_max), torch.where(pos_power, dt, torch.maximum(dt * f_dec, dt_min))))
    alpha.copy_(torch.where(grow, alpha * f_alpha, torch.where(pos_power, alpha, alpha_start)))
    velocities.mul_(keep[b].unsqueeze(-1)).add_(mix[b].unsqueeze(-1) * forces)


# ------------------------------------------------------------------------ segmented reductions
_MODES = {"sum": 0, "max": 1, "min": 2, "mean": 3}


def _segmented(values: torch.Tensor, idx: torch.Tensor, num_segments: int, mode: str) -> torch.Tensor:
    if _nat(values):
        return _nops.segmented_reduce(values, idx, int(num_segments), _MODES[mode])
    flat = values.reshape(values.shape[0], -1)
    ix = idx.long().unsqueeze(-1).expand_as(flat)
    out = torch.zeros(num_segments, flat.shape[1], dtype=flat.dtype, device=flat.device)
    if mode == "sum":
        out = out.double().scatter_add_(0, ix, flat.double()).to(flat.dtype)
    elif mode == "mean":
        cnt = torch.bincount(idx.long(), minlength=num_segments).clamp_min(1).unsqueeze(-1)
        out = (out.double().scatter_add_(0, ix, flat.double()) / cnt).to(flat.dtype)
    else:
        out = out.scatter_reduce(0, ix, flat, "amax" if mode == "max" else "amin", include_self=False)
    return out.reshape((num_segments,) + tuple(values.shape[1:]))


def segmented_sum(values, idx, num_segments):
    return _segmented(values, idx, num_segments, "sum")


def segmented_max(values, idx, num_segments):
    return _segmented(values, idx, num_segments, "max")


def segmented_min(values, idx, num_segments):
    return _segmented(values, idx, num_segments, "min")


def segmented_mean(values, idx, num_segments):
    return _segmented(values, idx, num_segments, "mean")


# ------------------------------------------------------------------------ cells
def compute_cell_inverse(cell: torch.Tensor) -> torch.Tensor:
    return torch.linalg.inv(cell)


def wrap_positions(positions, cell, batch_idx, pbc=None) -> torch.Tensor:
    """Positions wrapped into the cell along periodic directions (out of place)."""
    b = cell.shape[0]
    if pbc is None:
        pbc = torch.ones(b, 3, dtype=torch.bool, device=positions.device)
    inv = torch.linalg.inv(cell)
    if _nat(positions):
        return _nops.wrap_positions(positions.contiguous(), cell.contiguous(), inv.contiguous(),
                                                  pbc.contiguous(), _i32(batch_idx))
    bi = batch_idx.long()
    frac = torch.einsum("ni,nij->nj", positions, inv[bi])
    frac = torch.where(pbc[bi], frac - torch.floor(frac), frac)
    return torch.einsum("ni,nij->nj", frac, cell[bi])


def align_cell(positions, cell, batch_idx) -> None:
    """Rotate each system so its cell becomes lower-triangular (``a`` along x, ``b`` in xy); in place.

    Fractional coordinates are preserved.  Reference: ``nvalchemi/dynamics/_ops/cell_align.py:46-125``."""
    q, r = torch.linalg.qr(cell.transpose(-1, -2))  # cell^T = Q R  -> cell = R^T Q^T
    sign = torch.sign(torch.diagonal(r, dim1=-2, dim2=-1))
    sign = torch.where(sign == 0, torch.ones_like(sign), sign)
    q = q * sign.unsqueeze(-2)
    r = r * sign.unsqueeze(-1)
    new_cell = r.transpose(-1, -2)
    if _nat(positions) and positions.is_contiguous():
        _nops.affine_rows_(positions, q.contiguous(), None, None, None, None, None, _i32(batch_idx), False)  # r <- r Q
    else:
        positions.copy_(torch.einsum("ni,nij->nj", positions, q[batch_idx.long()]))
    cell.copy_(new_cell)


def batch_neighbor_list_rebuild_inplace(reference_positions, current_positions, batch_idx, rebuild_flags,
                                        skin_distance_threshold: float, update_reference_positions: bool, cell,
                                        cell_inv, pbc) -> None:
    """Set ``rebuild_flags[s]`` when any atom of system ``s`` moved more than the threshold (minimum image)."""
    if _nat(current_positions):
        _nops.neighbor_rebuild_check(reference_positions, current_positions.contiguous(), _i32(batch_idx),
                                                   rebuild_flags, float(skin_distance_threshold),
                                                   bool(update_reference_positions), cell.contiguous(),
                                                   cell_inv.contiguous(), pbc.contiguous())
        return
    bi = batch_idx.long()
    d = current_positions - reference_positions
    frac = torch.einsum("ni,nij->nj", d, cell_inv[bi])
    frac = torch.where(pbc[bi], frac - torch.floor(frac + 0.5), frac)
    d = torch.einsum("ni,nij->nj", frac, cell[bi])
    moved = (d * d).sum(-1) > skin_distance_threshold ** 2
    flags = torch.zeros_like(rebuild_flags).index_put_((bi,), moved, accumulate=True) if False else \
        torch.zeros(rebuild_flags.shape[0], dtype=torch.int32, device=d.device).index_add_(0, bi, moved.int()) > 0
    rebuild_flags.logical_or_(flags)
    if update_reference_positions:
        sel = rebuild_flags[bi]
        reference_positions[sel] = current_positions[sel]


# ------------------------------------------------------------------------ Nose-Hoover chains, barostat pieces
_YS_W = {1: [1.0], 3: [1.0 / (2.0 - 2.0 ** (1.0 / 3.0))] * 2, 5: [1.0 / (4.0 - 4.0 ** (1.0 / 3.0))] * 4}
_YS_W[3] = [_YS_W[3][0], 1.0 - 2.0 * _YS_W[3][0], _YS_W[3][0]]
_YS_W[5] = [_YS_W[5][0]] * 2 + [1.0 - 4.0 * _YS_W[5][0]] + [_YS_W[5][0]] * 2


def nhc_compute_masses(ndof: torch.Tensor, temperature: torch.Tensor, thermostat_time: torch.Tensor, chain_length: int
                       ) -> torch.Tensor:
    """``Q [M, C]``: ``Q_1 = N_f kT tau^2``, ``Q_k = kT tau^2`` (reference ``_ops/nose_hoover.py:65-127``)."""
    q = (temperature * thermostat_time ** 2).unsqueeze(1).repeat(1, chain_length)
    q[:, 0] = q[:, 0] * ndof
    return q.contiguous()


def _nhc_chain_torch(ke2, eta, eta_dot, Q, kT, ndof, dt, yoshida_order):
    c = eta.shape[1]
    scale = torch.ones_like(ke2)
    for w in _YS_W[yoshida_order]:
        h = w * dt
        for sweep in (range(c - 1, -1, -1), None, range(c)):
            if sweep is None:
                s = torch.exp(-0.5 * h * eta_dot[:, 0])
                scale = scale * s
                ke2.mul_(s * s)
                eta.add_(0.5 * h.unsqueeze(1) * eta_dot)
                continue
            for k in sweep:
                g = ((ke2 - ndof * kT) if k == 0 else (Q[:, k - 1] * eta_dot[:, k - 1] ** 2 - kT)) / Q[:, k]
                if k == c - 1:
                    eta_dot[:, k] += 0.25 * h * g
                else:
                    f = torch.exp(-0.125 * h * eta_dot[:, k + 1])
                    eta_dot[:, k] = (eta_dot[:, k] * f + 0.25 * h * g) * f
    return scale


def nhc_chain_scalar(ke2, eta, eta_dot, Q, temperature, ndof, dt, yoshida_order: int = 3) -> torch.Tensor:
    """Half-step propagation of one chain per system driven by ``ke2 = 2 KE`` (updated in place); returns the scale factor
    of the thermostatted velocities.  One kernel (thread = system) instead of ~150 tiny tensor operations."""
    if _nat(ke2) and eta.is_contiguous() and eta_dot.is_contiguous():
        return _nops.nhc_chain_scalar(ke2, eta, eta_dot, Q.contiguous(), temperature.contiguous(), ndof.contiguous(),
                                      dt.contiguous(), int(yoshida_order))
    return _nhc_chain_torch(ke2, eta, eta_dot, Q, temperature, ndof, dt, yoshida_order)


def nhc_chain_update(velocities, masses, eta, eta_dot, Q, temperature, dt, ndof, ke2, total_scale, step_scale=None,
                     dt_chain=None, batch_idx=None, compute_ke: bool = True, yoshida_order: int = 3) -> None:
    """Chain half step + velocity rescale (reference op ``nvalchemi::nhc_chain_update``).  ``compute_ke=False`` takes
    ``ke2`` as given (already summed over the ranks of a domain decomposition)."""
    m = eta.shape[0]
    if batch_idx is None:
        batch_idx = torch.zeros(velocities.shape[0], dtype=torch.int32, device=velocities.device)
    if _nat(velocities):
        empty = velocities.new_empty(0)
        _nops.nhc_chain_update(velocities, masses, eta, eta_dot, Q.contiguous(), temperature.contiguous(), dt.contiguous(),
                               ndof.contiguous(), ke2, total_scale, step_scale if step_scale is not None else empty,
                               dt_chain if dt_chain is not None else empty, _i32(batch_idx), bool(compute_ke),
                               int(yoshida_order))
        return
    if compute_ke:
        ke2.copy_(2.0 * compute_kinetic_energy(velocities, masses, batch_idx, m))
    total_scale.copy_(_nhc_chain_torch(ke2, eta, eta_dot, Q, temperature, ndof, dt, yoshida_order))
    velocities.mul_(total_scale[batch_idx.long()].unsqueeze(-1))


def nhc_velocity_half_step(velocities, forces, masses, dt, batch_idx) -> None:
    vv_velocity_finalize(velocities, forces, masses, dt, batch_idx)


def nhc_position_update(positions, velocities, dt, batch_idx) -> None:
    if _nat(positions):
        _nops.nhc_position_update(positions, velocities.contiguous(), dt, _i32(batch_idx))
        return
    positions.add_(velocities * dt[batch_idx.long()].unsqueeze(-1))


def compute_kinetic_tensor(velocities, masses, batch_idx, num_systems: int) -> torch.Tensor:
    """``sum_i m_i v_i (x) v_i`` per system, ``[M, 3, 3]`` (float64 accumulation)."""
    out = velocities.new_zeros(num_systems, 9)
    if _nat(velocities):
        _nops.compute_kinetic_tensor(velocities.contiguous(), masses, out, _i32(batch_idx))
    else:
        kt = (masses[:, None, None] * velocities[:, :, None] * velocities[:, None, :]).reshape(-1, 9).double()
        out.copy_(torch.zeros(num_systems, 9, dtype=torch.float64, device=out.device).index_add_(0, batch_idx.long(), kt))
    return out.reshape(num_systems, 3, 3)


def affine_rows_(x, A, batch_idx, y=None, C=None, forces=None, masses=None, kick=None, kick_first: bool = False) -> None:
    """``x_i <- x_i A_s + y_i C_s`` with an optional kick ``kick_s f_i / m_i`` added before (``kick_first``) or after the
    map; ``A, C [M, 3, 3]``, row-vector convention.  The per-atom primitive of the MTK barostat."""
    if _nat(x):
        _nops.affine_rows_(x, A.contiguous(), y, C, forces, masses, kick, _i32(batch_idx), bool(kick_first))
        return
    b = batch_idx.long()
    k = (kick[b] / masses).unsqueeze(-1) * forces if forces is not None else None
    v = x + k if (k is not None and kick_first) else x
    out = torch.einsum("ip,ipq->iq", v, A[b])
    if y is not None:
        out = out + torch.einsum("ip,ipq->iq", y, C[b])
    if k is not None and not kick_first:
        out = out + k
    x.copy_(out)


# ---- isobaric ensembles: functional pieces of the MTK integrators ----------------------------------------------------
# Reference op family ``dynamics/_ops/npt_nph.py:59-911``.  State is explicit (tensors in, tensors updated in place), so the
# same functions serve the NPT / NPH classes, user-written integrators and tests.  ``v_g`` is the 3 x 3 strain rate of the
# cell per system, ``coupling`` one of "isotropic" / "anisotropic" / "triclinic".
def compute_pressure_tensor(kinetic_tensors: torch.Tensor, stress: torch.Tensor, volumes: torch.Tensor) -> torch.Tensor:
    """``P = K / V - sigma`` per system (``K = sum m v (x) v``; ``sigma`` tensile positive, eV / A^3)."""
    return kinetic_tensors / volumes.reshape(-1, 1, 1) - stress.reshape(-1, 3, 3)


def compute_scalar_pressure(pressure_tensors: torch.Tensor) -> torch.Tensor:
    """``tr(P) / 3`` per system."""
    return torch.diagonal(pressure_tensors.reshape(-1, 3, 3), dim1=1, dim2=2).sum(-1) / 3.0


def compute_barostat_mass(ndof: torch.Tensor, kT: torch.Tensor, barostat_time: torch.Tensor) -> torch.Tensor:
    """``W = (N_f + 3) kT tau_b^2`` (Martyna-Tobias-Klein)."""
    return (ndof + 3.0) * kT * barostat_time ** 2


def project_cell_force(g: torch.Tensor, coupling: str) -> torch.Tensor:
    """Restrict a 3 x 3 generalised force to the degrees of freedom of the coupling mode (identity multiple, diagonal,
    symmetric)."""
    if coupling == "triclinic":
        return 0.5 * (g + g.transpose(-1, -2))
    d = torch.diagonal(g, dim1=1, dim2=2)
    if coupling == "isotropic":
        d = d.mean(-1, keepdim=True).expand(-1, 3)
    elif coupling != "anisotropic":
        raise ValueError("coupling must be 'isotropic', 'anisotropic' or 'triclinic'")
    return torch.diag_embed(d)


def npt_barostat_half_step(v_g: torch.Tensor, pressure_tensors: torch.Tensor, target_pressure: torch.Tensor, volumes: torch.Tensor,
                           ke2: torch.Tensor, ndof: torch.Tensor, barostat_mass: torch.Tensor, dt: torch.Tensor,
                           coupling: str = "isotropic") -> torch.Tensor:
    """``v_g += dt/2 [V (P - p_ext 1) + (2 KE / N_f) 1] / W``, projected on the coupling mode; in place, returns ``v_g``."""
    eye = torch.eye(3, dtype=v_g.dtype, device=v_g.device)
    g = volumes.reshape(-1, 1, 1) * (pressure_tensors - target_pressure.reshape(-1, 1, 1) * eye) + (ke2 / ndof).reshape(-1, 1, 1) * eye
    return v_g.add_(0.5 * dt.reshape(-1, 1, 1) * project_cell_force(g, coupling) / barostat_mass.reshape(-1, 1, 1))


nph_barostat_half_step = npt_barostat_half_step


def npt_cell_damping(v_g: torch.Tensor, ndof: torch.Tensor, dt: torch.Tensor) -> torch.Tensor:
    """``exp(-dt/2 (v_g + tr(v_g) / N_f 1))`` per system: what the cell motion does to the particle velocities."""
    tr = torch.diagonal(v_g, dim1=1, dim2=2).sum(-1) / ndof
    eye = torch.eye(3, dtype=v_g.dtype, device=v_g.device)
    return torch.linalg.matrix_exp(-0.5 * dt.reshape(-1, 1, 1) * (v_g + tr.reshape(-1, 1, 1) * eye))


def npt_velocity_half_step(velocities: torch.Tensor, forces: torch.Tensor, masses: torch.Tensor, v_g: torch.Tensor,
                           ndof: torch.Tensor, dt: torch.Tensor, batch_idx: torch.Tensor, kick_first: bool = False) -> None:
    """Damping by the cell motion and the half kick ``v += dt/2 F/m`` in one per-atom kernel (``kick_first`` mirrors the
    order for the opening half of a step)."""
    affine_rows_(velocities, npt_cell_damping(v_g, ndof, dt), batch_idx, forces=forces, masses=masses, kick=0.5 * dt,
                 kick_first=kick_first)


nph_velocity_half_step = npt_velocity_half_step


def npt_position_update(positions: torch.Tensor, velocities: torch.Tensor, v_g: torch.Tensor, dt: torch.Tensor,
                        batch_idx: torch.Tensor) -> torch.Tensor:
    """``r <- r exp(dt v_g) + dt v exp(dt v_g / 2)`` (one per-atom kernel); returns ``exp(dt v_g)`` for the cell update."""
    d = dt.reshape(-1, 1, 1)
    grow = torch.linalg.matrix_exp(d * v_g)
    affine_rows_(positions, grow, batch_idx, y=velocities, C=d * torch.linalg.matrix_exp(0.5 * d * v_g))
    return grow


def npt_cell_update(cell: torch.Tensor, grow: torch.Tensor) -> torch.Tensor:
    """Lattice vectors (rows) follow the same map as the positions: ``h <- h exp(dt v_g)``; in place."""
    c = cell.reshape(-1, 3, 3)
    c.copy_(c @ grow)
    return cell


def npt_thermostat_half_step(velocities: torch.Tensor, masses: torch.Tensor, batch_idx: torch.Tensor, v_g: torch.Tensor,
                             state: dict, ndof: torch.Tensor, barostat_mass: torch.Tensor, coupling: str, chain_length: int,
                             ke_reduce: Any = None) -> None:
    """Half step of the two Nose-Hoover chains: particles (``eta`` / ``eta_dot``) and barostat (``xi`` / ``xi_dot``).
    ``state`` holds ``kT, tau_t, tau_b, dt`` and the chain variables; velocities and ``v_g`` are scaled in place."""
    m = ndof.shape[0]
    ke2 = 2.0 * compute_kinetic_energy(velocities, masses, batch_idx, m)
    if ke_reduce is not None:
        ke2 = ke_reduce(ke2)
    Q = nhc_compute_masses(ndof, state["kT"], state["tau_t"], chain_length)
    velocity_rescale(velocities, nhc_chain_scalar(ke2, state["eta"], state["eta_dot"], Q, state["kT"], ndof, state["dt"]), batch_idx)
    n_b = torch.full_like(ndof, {"isotropic": 1.0, "anisotropic": 3.0, "triclinic": 6.0}[coupling])
    kb2 = barostat_mass * (v_g ** 2).sum((-1, -2)) * (1.0 / 3.0 if coupling == "isotropic" else 1.0)
    Qb = nhc_compute_masses(n_b, state["kT"], state["tau_b"], chain_length)
    v_g.mul_(nhc_chain_scalar(kb2, state["xi"], state["xi_dot"], Qb, state["kT"], n_b, state["dt"]).reshape(-1, 1, 1))


def stress_to_cell_force(cell: torch.Tensor, stress: torch.Tensor, factor: torch.Tensor | float = 1.0) -> torch.Tensor:
    """Generalised force on the lattice vectors for variable-cell relaxation: ``dE/d(strain) = V sigma`` (sigma tensile
    positive), so the force on the cell rows is ``-V h sigma / factor`` (``factor`` balances cell against atomic degrees of
    freedom, typically the atom count)."""
    c, s = cell.reshape(-1, 3, 3), stress.reshape(-1, 3, 3)
    vol = torch.linalg.det(c).abs()
    f = factor if isinstance(factor, torch.Tensor) else torch.full_like(vol, float(factor))
    return -(vol[:, None, None] * torch.matmul(c, s)) / f[:, None, None]
