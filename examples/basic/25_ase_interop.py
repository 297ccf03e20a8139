# SPDX-License-Identifier: Apache-2.0
"""Round trip with ASE: ``AtomicData.from_atoms`` reads anything that looks like ``ase.Atoms`` (numbers, positions, cell,
pbc, masses, velocities, initial charges) and ``to_atoms`` writes one back.  Without ASE installed the script uses a
minimal stand-in with the same accessor names, which is all ``from_atoms`` relies on."""
import numpy as np
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch
from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

try:
    from ase.build import bulk

    atoms = bulk("Ar", "fcc", a=5.26, cubic=True).repeat((2, 2, 2))
    have_ase = True
except ImportError:
    have_ase = False

    class Atoms:  # the accessors from_atoms looks for
        def __init__(self, numbers, positions, cell, pbc):
            self._z, self._r, self._cell, self._pbc = np.asarray(numbers), np.asarray(positions, float), np.asarray(cell, float), pbc

        def get_atomic_numbers(self): return self._z
        def get_positions(self): return self._r
        def get_cell(self): return self._cell
        def get_pbc(self): return np.asarray(self._pbc)
        def get_masses(self): return np.full(len(self._z), 39.948)
        def get_velocities(self): return None

    base = np.array([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]])
    grid = np.stack(np.meshgrid(*(np.arange(2),) * 3, indexing="ij"), -1).reshape(-1, 1, 3)
    atoms = Atoms([18] * 32, ((grid + base).reshape(-1, 3)) * 5.26, np.eye(3) * 10.52, [True] * 3)

rng = np.random.default_rng(0)
data = AtomicData.from_atoms(atoms, dtype=torch.float64)
data.positions.add_(torch.as_tensor(rng.normal(0, 0.08, size=tuple(data.positions.shape))))
batch = Batch.from_data_list([data])
model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.5, switch_width=1.0)
relax = FIRE(model, dt=1.0, convergence_hook=ConvergenceHook.from_fmax(1e-3), hooks=model.make_neighbor_hooks())
relax.run(batch, n_steps=300)
fmax = float(batch.forces.norm(dim=-1).max())
print(f"{'ase.Atoms' if have_ase else 'stand-in Atoms'} -> AtomicData ({data.num_nodes} atoms) -> FIRE: fmax = {fmax:.2e} eV/A after {relax.step_count} steps")
if have_ase:
    back = batch.get_data(0).to_atoms()
    print("back to ASE:", back.get_chemical_formula(), "cell", np.round(back.get_cell().lengths(), 3))
assert fmax < 5e-3
