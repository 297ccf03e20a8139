# SPDX-License-Identifier: Apache-2.0
"""Operator names of the reference under ``torch.ops.nvalchemi`` / ``torch.ops.nvalchemi_hooks``.

The reference registers its kernels as torch custom ops (``@torch.library.custom_op`` over NVIDIA Warp kernels) and
user code may call them by name.  The hot ones are native operators of this package's extension already
(``vv_position_update``, ``langevin_half_step``, ``lj_energy_forces_virial_batch`` ...).  This module registers the
remaining names as thin operators over this package's implementations, so the same call sites keep working:
``import nvalchemi_toolkit_b200.ops.compat`` (done by ``nvalchemi_toolkit_b200.ops``).  In-place semantics follow the
reference: the ops mutate their first arguments and return nothing.
"""
from __future__ import annotations

import torch

from nvalchemi_toolkit_b200.dynamics import _ops

_lib = torch.library.Library("nvalchemi", "FRAGMENT")
_hooks = torch.library.Library("nvalchemi_hooks", "DEF")
_registered: list[str] = []


def _define(lib: torch.library.Library, schema: str, fn) -> None:
    name = schema.split("(")[0]
    lib.define(schema)
    lib.impl(name, fn, "CompositeExplicitAutograd")
    _registered.append(name)


def _initialize_velocities(velocities, masses, temperature, batch_idx, random_seed=42, remove_com=True,
                           remove_rotations=False, rescale=True, positions=None):
    _ops.initialize_velocities(velocities, masses, temperature, batch_idx, random_seed=random_seed, remove_com=remove_com,
                               remove_rotations=remove_rotations, rescale=rescale, positions=positions)


def _lj_energy_forces_batch(positions, cells, neighbor_matrix, neighbor_matrix_shifts, num_neighbors, batch_idx, fill_value,
                            epsilon, sigma, cutoff, switch_width, half_list, num_systems):
    from nvalchemi_toolkit_b200.models.lj import lj_energy_forces_virial_batch

    e, f, _ = lj_energy_forces_virial_batch(positions, cells, neighbor_matrix, neighbor_matrix_shifts, num_neighbors,
                                            batch_idx, fill_value, epsilon, sigma, cutoff, switch_width, half_list, num_systems)
    return e, f


def _per_system_reduce(local_vals, system_index, n_systems):
    import torch.distributed as dist

    out = _ops.segmented_sum(local_vals, system_index, n_systems)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(out)
    return out


_define(_lib, "initialize_velocities(Tensor(a!) velocities, Tensor masses, Tensor temperature, Tensor batch_idx, int random_seed=42, bool remove_com=True, bool remove_rotations=False, bool rescale=True, Tensor? positions=None) -> ()",
        _initialize_velocities)
_define(_lib, "remove_com_motion(Tensor(a!) velocities, Tensor masses, Tensor batch_idx, int num_systems) -> ()",
        lambda v, m, b, n: _ops.remove_com_motion(v, m, b, n))
_define(_lib, "velocity_rescale(Tensor(a!) velocities, Tensor scale_factor, Tensor batch_idx) -> ()",
        lambda v, s, b: _ops.velocity_rescale(v, s, b))
_define(_lib, "compute_temperature(Tensor kinetic_energy, Tensor num_atoms_per_system) -> Tensor",
        lambda ke, n: _ops.compute_temperature(ke, n))
_define(_lib, "align_cell(Tensor(a!) positions, Tensor(b!) cell, Tensor batch_idx) -> ()",
        lambda p, c, b: _ops.align_cell(p, c, b))
_define(_lib, "_batch_neighbor_list_rebuild_inplace(Tensor(a!) reference_positions, Tensor current_positions, Tensor batch_idx, Tensor(b!) rebuild_flags, float skin_distance_threshold, bool update_reference_positions, Tensor cell, Tensor cell_inv, Tensor pbc) -> ()",
        lambda r, c, b, f, t, u, cell, inv, pbc: _ops.batch_neighbor_list_rebuild_inplace(r, c, b, f, t, u, cell, inv, pbc))
_define(_lib, "lj_energy_forces_batch(Tensor positions, Tensor cells, Tensor neighbor_matrix, Tensor neighbor_matrix_shifts, Tensor num_neighbors, Tensor batch_idx, int fill_value, float epsilon, float sigma, float cutoff, float switch_width, bool half_list, int num_systems) -> (Tensor, Tensor)",
        _lj_energy_forces_batch)
_define(_lib, "per_system_reduce(Tensor local_vals, Tensor system_index, int n_systems) -> Tensor", _per_system_reduce)
for _mode in ("sum", "max", "min", "mean"):
    _define(_hooks, f"segmented_{_mode}(Tensor values, Tensor idx, int num_segments) -> Tensor",
            (lambda mode: lambda v, i, n: _ops._segmented(v, i, n, mode))(_mode))
_define(_hooks, "compute_kinetic_energy(Tensor velocities, Tensor masses, Tensor batch_idx, int num_graphs) -> Tensor",
        lambda v, m, b, n: _ops.compute_kinetic_energy(v, m, b, n))
_define(_hooks, "wrap_positions(Tensor positions, Tensor cell, Tensor batch_idx) -> Tensor",
        lambda p, c, b: _ops.wrap_positions(p, c, b))


def registered_names() -> list[str]:
    return list(_registered)
