# SPDX-License-Identifier: Apache-2.0
"""``AtomicData``: one atomistic system as a validated graph of tensors.

Field names, level classification (node / edge / system) and validator
behaviour follow the reference's ``nvalchemi/data/atomic_data.py:103-1196``:
consistent node/edge counts, floating tensors cast to the dtype of
``positions`` (with a warning), default masses, categories and velocities, and
all tensors moved to one device.  System-level tensors are normalised to carry
a leading axis of length 1 (``cell [1,3,3]``, ``pbc [1,3]``, ``energy [1,1]``)
so that batching is a plain concatenation.
"""
from __future__ import annotations

import hashlib
import warnings
from typing import Annotated, Any, ClassVar

import numpy as np
import torch
from pydantic import BaseModel, BeforeValidator, ConfigDict, Field, PlainSerializer, model_validator

from nvalchemi_toolkit_b200._serialization import tensor_from_json, tensor_to_json
from nvalchemi_toolkit_b200._typing import AtomCategory
from nvalchemi_toolkit_b200.utils.elements import ATOMIC_MASSES, SYMBOL_TO_Z


def _coerce_tensor(v: Any) -> Any:
    if v is None or isinstance(v, torch.Tensor):
        return v
    if isinstance(v, dict) and "data" in v:
        return tensor_from_json(v)
    if isinstance(v, np.ndarray):
        return torch.from_numpy(v)
    if isinstance(v, (list, tuple)) and v and isinstance(v[0], AtomCategory):
        return torch.tensor([c.value for c in v], dtype=torch.long)
    return torch.as_tensor(v)


TensorField = Annotated[
    torch.Tensor | None,
    BeforeValidator(_coerce_tensor),
    PlainSerializer(tensor_to_json, when_used="json"),
]


def _opt(desc: str) -> Any:
    return Field(default=None, description=desc)


class DataMixin:
    """Dictionary-style access shared by ``AtomicData`` and ``Batch``."""

    def __getitem__(self, key: str) -> Any:
        return getattr(self, key)

    def __setitem__(self, key: str, value: Any) -> None:
        setattr(self, key, value)

    def get(self, key: str, default: Any = None) -> Any:
        val = getattr(self, key, None)
        return default if val is None else val


class AtomicData(BaseModel, DataMixin):
    """A single molecular or periodic system.

    Required: ``atomic_numbers [V]`` and ``positions [V,3]``.  Everything else
    is optional; see the class-level key sets for which axis each field is
    batched along.
    """

    model_config: ClassVar[ConfigDict] = ConfigDict(
        arbitrary_types_allowed=True, validate_assignment=False, extra="allow"
    )

    atomic_numbers: Annotated[
        torch.Tensor, BeforeValidator(_coerce_tensor), PlainSerializer(tensor_to_json, when_used="json")
    ] = Field(description="Atomic numbers [V]")
    positions: Annotated[
        torch.Tensor, BeforeValidator(_coerce_tensor), PlainSerializer(tensor_to_json, when_used="json")
    ] = Field(description="Cartesian coordinates [V,3] (Angstrom)")
    atomic_masses: TensorField = _opt("Atomic masses [V] (amu)")
    atom_categories: TensorField = _opt("AtomCategory value per atom [V]")
    neighbor_list: TensorField = _opt("COO neighbour list [E,2] = (source, target)")
    shifts: TensorField = _opt("Cartesian image displacement per edge [E,3]")
    neighbor_list_shifts: TensorField = _opt("Integer lattice image per edge [E,3]")
    neighbor_matrix: TensorField = _opt("Dense neighbour matrix [V,K]")
    neighbor_matrix_shifts: TensorField = _opt("Integer images of the matrix [V,K,3]")
    num_neighbors: TensorField = _opt("Valid neighbours per atom [V]")
    cell: TensorField = _opt("Lattice vectors as rows [1,3,3]")
    pbc: TensorField = _opt("Periodic directions [1,3] bool")
    forces: TensorField = _opt("Forces [V,3] (eV/Angstrom)")
    energy: TensorField = _opt("Total energy [1,1] (eV)")
    stress: TensorField = _opt("Tensile-positive Cauchy stress [1,3,3] (eV/A^3)")
    virial: TensorField = _opt("Virial W = -dE/d(strain) [1,3,3] (eV)")
    dipole: TensorField = _opt("Dipole [1,3]")
    charges: TensorField = _opt("Partial charges [V]")
    charge: TensorField = _opt("Total charge [1,1]")
    node_attrs: TensorField = _opt("Node attributes [V,F]")
    node_alpha_spins: TensorField = _opt("Alpha spins [V,1]")
    node_beta_spins: TensorField = _opt("Beta spins [V,1]")
    spin: TensorField = _opt("Spin / multiplicity [1,1]")
    graph_alpha_spins: TensorField = _opt("Graph alpha spins [1,1]")
    node_embeddings: TensorField = _opt("Node embeddings [V,H]")
    edge_embeddings: TensorField = _opt("Edge embeddings [E,H]")
    graph_embeddings: TensorField = _opt("Graph embeddings [1,H]")
    velocities: TensorField = _opt("Velocities [V,3]")
    momenta: TensorField = _opt("Momenta [V,3]")
    kinetic_energies: TensorField = _opt("Per-atom kinetic energies [V,1]")
    info: dict[str, Any] = Field(default_factory=dict)

    _default_node_keys: ClassVar[frozenset[str]] = frozenset({
        "atomic_masses", "positions", "forces", "charges", "node_embeddings", "atomic_numbers",
        "node_attrs", "node_alpha_spins", "node_beta_spins", "atom_categories", "velocities",
        "momenta", "kinetic_energies", "neighbor_matrix", "neighbor_matrix_shifts", "num_neighbors",
    })
    _default_edge_keys: ClassVar[frozenset[str]] = frozenset(
        {"shifts", "neighbor_list_shifts", "neighbor_list", "edge_embeddings"}
    )
    _default_system_keys: ClassVar[frozenset[str]] = frozenset(
        {"energy", "stress", "virial", "dipole", "charge", "graph_embeddings", "cell", "pbc", "spin",
         "graph_alpha_spins"}
    )
    # trailing shape each system-level field is normalised to (after the leading 1)
    _system_shapes: ClassVar[dict[str, tuple[int, ...]]] = {
        "cell": (3, 3), "pbc": (3,), "energy": (1,), "stress": (3, 3), "virial": (3, 3),
        "dipole": (3,), "charge": (1,), "spin": (1,), "graph_alpha_spins": (1,),
    }

    # ------------------------------------------------------------------ init
    def model_post_init(self, __context: Any) -> None:
        extra_node = set(getattr(self, "__node_keys__", ()))
        extra_edge = set(getattr(self, "__edge_keys__", ()))
        extra_sys = set(getattr(self, "__system_keys__", ()))
        object.__setattr__(self, "__node_keys__", set(self._default_node_keys) | extra_node)
        object.__setattr__(self, "__edge_keys__", set(self._default_edge_keys) | extra_edge)
        object.__setattr__(self, "__system_keys__", set(self._default_system_keys) | extra_sys)

    @model_validator(mode="after")
    def _normalise(self) -> "AtomicData":
        d = self.__dict__
        if self.atomic_numbers.dim() != 1:
            raise ValueError("atomic_numbers must be 1-D [V]")
        if self.positions.dim() != 2 or self.positions.shape[-1] != 3:
            raise ValueError("positions must have shape [V,3]")
        if not self.positions.dtype.is_floating_point:
            d["positions"] = self.positions.to(torch.get_default_dtype())
        d["atomic_numbers"] = self.atomic_numbers.long()
        n = self.atomic_numbers.shape[0]
        if self.positions.shape[0] != n:
            raise ValueError(
                f"Inconsistent number of atoms in positions: expected {n}, got {self.positions.shape[0]}"
            )
        # device: promote everything to an accelerator if either anchor lives there
        devs = {self.atomic_numbers.device, self.positions.device}
        target = next((dv for dv in devs if dv.type != "cpu"), torch.device("cpu"))
        dtype = self.positions.dtype
        # system-level shape normalisation
        for key, tail in self._system_shapes.items():
            v = d.get(key)
            if isinstance(v, torch.Tensor):
                if key == "pbc":
                    v = v.to(torch.bool)
                numel = int(np.prod(tail))
                if v.numel() == numel:
                    v = v.reshape((1,) + tail)
                d[key] = v
        casted: list[str] = []
        extras = self.__pydantic_extra__ or {}
        for store in (d, extras):
            for key, v in list(store.items()):
                if not isinstance(v, torch.Tensor):
                    continue
                if v.dtype.is_floating_point and v.dtype != dtype:
                    v = v.to(dtype)
                    casted.append(key)
                if v.device != target:
                    v = v.to(target)
                store[key] = v
        if casted:
            warnings.warn(
                f"AtomicData fields {sorted(casted)} were cast from their original dtypes to {dtype} "
                "to match positions. Pass tensors with matching dtypes to silence this warning.",
                UserWarning, stacklevel=3,
            )
        # defaults
        if d.get("atomic_masses") is None:
            table = ATOMIC_MASSES.to(device=target, dtype=dtype)
            d["atomic_masses"] = table[d["atomic_numbers"].clamp(0, table.numel() - 1)]
        if d.get("atom_categories") is None:
            d["atom_categories"] = torch.zeros(n, dtype=torch.long, device=target)
        else:
            d["atom_categories"] = d["atom_categories"].long()
        if d.get("velocities") is None:
            d["velocities"] = torch.zeros_like(d["positions"])
        # count consistency
        node_keys = d.get("__node_keys__", self._default_node_keys)
        for key in node_keys:
            v = d.get(key, extras.get(key))
            if isinstance(v, torch.Tensor) and v.shape[0] != n:
                raise ValueError(f"Inconsistent number of atoms in {key}: expected {n}, got {v.shape[0]}")
        nl = d.get("neighbor_list")
        if isinstance(nl, torch.Tensor):
            ne = nl.shape[0]
            for key in d.get("__edge_keys__", self._default_edge_keys):
                v = d.get(key, extras.get(key))
                if isinstance(v, torch.Tensor) and v.shape[0] != ne:
                    raise ValueError(f"Inconsistent number of edges in {key}: expected {ne}, got {v.shape[0]}")
        return self

    # ------------------------------------------------------------ properties
    @property
    def device(self) -> torch.device:
        return self.positions.device

    @property
    def dtype(self) -> torch.dtype:
        return self.positions.dtype

    @property
    def num_nodes(self) -> int:
        return int(self.atomic_numbers.shape[0])

    @property
    def num_edges(self) -> int:
        return 0 if self.neighbor_list is None else int(self.neighbor_list.shape[0])

    def _tensor_items(self) -> dict[str, torch.Tensor]:
        out = {k: v for k, v in self.__dict__.items() if isinstance(v, torch.Tensor)}
        for k, v in (self.__pydantic_extra__ or {}).items():
            if isinstance(v, torch.Tensor):
                out[k] = v
        return out

    def _level_items(self, keys: set[str]) -> dict[str, torch.Tensor]:
        return {k: v for k, v in self._tensor_items().items() if k in keys}

    @property
    def node_properties(self) -> dict[str, torch.Tensor]:
        return self._level_items(self.__node_keys__)

    @property
    def edge_properties(self) -> dict[str, torch.Tensor]:
        return self._level_items(self.__edge_keys__)

    @property
    def system_properties(self) -> dict[str, torch.Tensor]:
        return self._level_items(self.__system_keys__)

    def level_of(self, key: str) -> str | None:
        if key in self.__node_keys__:
            return "node"
        if key in self.__edge_keys__:
            return "edge"
        if key in self.__system_keys__:
            return "system"
        return None

    def _claim(self, key: str, level: str) -> None:
        """A field lives on ONE level: registering a name that another level already owns (built-in fields included,
        e.g. the per-system ``spin`` or ``charge``) would make batches collate it twice with different shapes."""
        current = self.level_of(key)
        if current is not None and current != level:
            raise ValueError(f"'{key}' is already a {current}-level field; choose another name for the {level}-level quantity")

    def add_node_property(self, key: str, value: torch.Tensor, node_dim: int = 0) -> None:
        self._claim(key, "node")
        if value.shape[node_dim] != self.num_nodes:
            raise ValueError(f"{key}: expected {self.num_nodes} rows, got {value.shape[node_dim]}")
        object.__setattr__(self, key, value) if key in type(self).model_fields else self._set_extra(key, value)
        self.__node_keys__.add(key)

    def add_edge_property(self, key: str, value: torch.Tensor) -> None:
        self._claim(key, "edge")
        object.__setattr__(self, key, value) if key in type(self).model_fields else self._set_extra(key, value)
        self.__edge_keys__.add(key)

    def add_system_property(self, key: str, value: torch.Tensor) -> None:
        self._claim(key, "system")
        object.__setattr__(self, key, value) if key in type(self).model_fields else self._set_extra(key, value)
        self.__system_keys__.add(key)

    def _set_extra(self, key: str, value: Any) -> None:
        if self.__pydantic_extra__ is None:
            object.__setattr__(self, "__pydantic_extra__", {})
        self.__pydantic_extra__[key] = value

    # ---------------------------------------------------------------- moves
    def to(self, device: torch.device | str | None = None, dtype: torch.dtype | None = None,
           non_blocking: bool = False) -> "AtomicData":
        kw: dict[str, Any] = {}
        for k, v in self._tensor_items().items():
            if dtype is not None and v.dtype.is_floating_point:
                v = v.to(dtype)
            if device is not None:
                v = v.to(device, non_blocking=non_blocking)
            kw[k] = v
        kw["info"] = dict(self.info)
        new = type(self).model_construct(**kw)
        new.model_post_init(None)
        for lvl in ("__node_keys__", "__edge_keys__", "__system_keys__"):
            getattr(new, lvl).update(getattr(self, lvl))
        return new

    def clone(self) -> "AtomicData":
        kw = {k: v.clone() for k, v in self._tensor_items().items()}
        kw["info"] = dict(self.info)
        new = type(self).model_construct(**kw)
        new.model_post_init(None)
        for lvl in ("__node_keys__", "__edge_keys__", "__system_keys__"):
            getattr(new, lvl).update(getattr(self, lvl))
        return new

    # ------------------------------------------------------------- builders
    @classmethod
    def from_atoms(cls, atoms: Any, dtype: torch.dtype = torch.float32, device: str | torch.device = "cpu",
                   **extra: Any) -> "AtomicData":
        """Build from an ASE ``Atoms``-like object (duck-typed: ``get_atomic_numbers``,
        ``get_positions``, ``get_cell``, ``get_pbc``, optional ``get_masses`` / velocities).

        Reference: ``data/atomic_data.py`` ``from_atoms``.
        """
        kw: dict[str, Any] = {
            "atomic_numbers": torch.as_tensor(np.asarray(atoms.get_atomic_numbers()), dtype=torch.long),
            "positions": torch.as_tensor(np.asarray(atoms.get_positions()), dtype=dtype),
        }
        cell = np.asarray(atoms.get_cell()) if hasattr(atoms, "get_cell") else None
        pbc = np.asarray(atoms.get_pbc()) if hasattr(atoms, "get_pbc") else None
        if cell is not None and np.abs(cell).sum() > 0:
            kw["cell"] = torch.as_tensor(cell, dtype=dtype).reshape(1, 3, 3)
            kw["pbc"] = torch.as_tensor(pbc if pbc is not None else [False] * 3, dtype=torch.bool).reshape(1, 3)
        if hasattr(atoms, "get_masses"):
            kw["atomic_masses"] = torch.as_tensor(np.asarray(atoms.get_masses()), dtype=dtype)
        if hasattr(atoms, "get_velocities") and atoms.get_velocities() is not None:
            # ASE velocities are in Angstrom / (ASE time unit) = sqrt(eV/amu): already internal units
            kw["velocities"] = torch.as_tensor(np.asarray(atoms.get_velocities()), dtype=dtype)
        if hasattr(atoms, "get_initial_charges"):
            q = np.asarray(atoms.get_initial_charges())
            if np.any(q != 0):
                kw["charges"] = torch.as_tensor(q, dtype=dtype)
        kw.update(extra)
        return cls(**kw).to(device)

    def to_atoms(self) -> Any:
        """An ``ase.Atoms`` with positions, cell, pbc, masses, velocities (needs ``ase``)."""
        from nvalchemi_toolkit_b200._optional import OptionalDependency

        ase = OptionalDependency.ASE.import_module()
        kw: dict[str, Any] = {"numbers": self.atomic_numbers.cpu().numpy(), "positions": self.positions.detach().cpu().numpy()}
        if getattr(self, "cell", None) is not None:
            kw["cell"] = self.cell.detach().reshape(3, 3).cpu().numpy()
            kw["pbc"] = self.pbc.reshape(3).cpu().numpy() if getattr(self, "pbc", None) is not None else False
        atoms = ase.Atoms(**kw)
        if getattr(self, "atomic_masses", None) is not None:
            atoms.set_masses(self.atomic_masses.detach().cpu().numpy())
        if getattr(self, "velocities", None) is not None:
            atoms.set_velocities(self.velocities.detach().cpu().numpy())
        return atoms

    @classmethod
    def from_structure(cls, structure: Any, dtype: torch.dtype = torch.float32,
                       device: str | torch.device = "cpu", **extra: Any) -> "AtomicData":
        """Build from a pymatgen ``Structure``/``Molecule``-like object (duck-typed)."""
        kw: dict[str, Any] = {
            "atomic_numbers": torch.as_tensor(list(structure.atomic_numbers), dtype=torch.long),
            "positions": torch.as_tensor(np.asarray(structure.cart_coords), dtype=dtype),
        }
        lattice = getattr(structure, "lattice", None)
        if lattice is not None:
            kw["cell"] = torch.as_tensor(np.asarray(lattice.matrix), dtype=dtype).reshape(1, 3, 3)
            kw["pbc"] = torch.tensor([[True, True, True]])
        kw.update(extra)
        return cls(**kw).to(device)

    @classmethod
    def from_symbols(cls, symbols: list[str], positions: Any, **kw: Any) -> "AtomicData":
        z = torch.tensor([SYMBOL_TO_Z[s] for s in symbols], dtype=torch.long)
        return cls(atomic_numbers=z, positions=torch.as_tensor(positions), **kw)

    # --------------------------------------------------------------- hashing
    @property
    def chemical_hash(self) -> str:
        """BLAKE2s digest invariant to atom ordering; sensitive to cell / pbc when set."""
        z = self.atomic_numbers.cpu().numpy()
        pos = self.positions.detach().cpu().double().numpy()
        order = np.lexsort((np.round(pos[:, 2], 6), np.round(pos[:, 1], 6), np.round(pos[:, 0], 6), z))
        h = hashlib.blake2s()
        h.update(np.ascontiguousarray(z[order]).astype(np.int64).tobytes())
        h.update(np.round(pos[order], 6).tobytes())
        if self.pbc is not None and self.cell is not None:
            h.update(self.pbc.cpu().numpy().astype(np.uint8).tobytes())
            h.update(np.round(self.cell.detach().cpu().double().numpy(), 6).tobytes())
        return h.hexdigest()

    # --------------------------------------------------------------- helpers
    def to_one_hot(self, z_table: list[int] | torch.Tensor) -> torch.Tensor:
        """One-hot ``[V, len(z_table)]`` of ``atomic_numbers`` against a table of Z values."""
        table = torch.as_tensor(z_table, device=self.device, dtype=torch.long)
        hit = self.atomic_numbers[:, None] == table[None, :]
        if not bool(hit.any(dim=1).all()):
            raise ValueError("atomic_numbers contains elements missing from z_table")
        return hit.to(self.dtype)

    @staticmethod
    def voigt_to_matrix(v: torch.Tensor) -> torch.Tensor:
        """Voigt ``[...,6] = (xx,yy,zz,yz,xz,xy)`` (or ``[...,9]`` / ``[...,3,3]``) to ``[...,3,3]``."""
        if v.shape[-2:] == (3, 3):
            return v
        if v.shape[-1] == 9:
            return v.reshape(*v.shape[:-1], 3, 3)
        if v.shape[-1] != 6:
            raise ValueError("expected a Voigt vector of length 6")
        xx, yy, zz, yz, xz, xy = v.unbind(-1)
        return torch.stack([xx, xy, xz, xy, yy, yz, xz, yz, zz], dim=-1).reshape(*v.shape[:-1], 3, 3)

    def __repr__(self) -> str:  # short: tensors are summarised by shape
        parts = [f"{k}={tuple(v.shape)}" for k, v in sorted(self._tensor_items().items())]
        return f"AtomicData({', '.join(parts)})"
