# SPDX-License-Identifier: Apache-2.0
"""Columnar storage for batches of variable-size systems.

Three pieces (same roles as the reference's ``nvalchemi/data/level_storage.py:225-2491``,
built on plain dictionaries of tensors instead of TensorDict):

* :class:`UniformLevelStorage` — one row per system (``cell``, ``energy`` ...).
* :class:`SegmentedLevelStorage` — concatenated rows with per-system segment
  lengths (``positions``, ``neighbor_list`` ...); ``batch_ptr`` / ``batch_idx``
  are int32 and derived lazily.
* :class:`MultiLevelStorage` — routes an attribute name to its group through a
  :class:`LevelSchema`.

Storages may be allocated with spare capacity (fixed-size GPU buffers).  Valid
data is always kept compact at the front: ``put`` appends systems that fit,
``defrag`` removes systems and closes the gaps, both without changing capacity.
The row copies go through :mod:`nvalchemi_toolkit_b200.ops.buffer` (CUDA
kernels on GPU tensors, vectorised torch on CPU).
"""
from __future__ import annotations

from typing import Any, Iterable, Iterator, Mapping

import torch

from nvalchemi_toolkit_b200.ops import buffer as _buf

_NODE_DEFAULT = frozenset({
    "atomic_masses", "positions", "forces", "charges", "node_embeddings", "atomic_numbers", "node_attrs",
    "node_alpha_spins", "node_beta_spins", "atom_categories", "velocities", "momenta", "kinetic_energies",
    "neighbor_matrix", "neighbor_matrix_shifts", "num_neighbors",
})
_EDGE_DEFAULT = frozenset({"shifts", "neighbor_list_shifts", "neighbor_list", "edge_embeddings"})
_SYSTEM_DEFAULT = frozenset({
    "energy", "stress", "virial", "dipole", "charge", "graph_embeddings", "cell", "pbc", "spin",
    "graph_alpha_spins", "status", "system_id",
})
GROUPS = ("atoms", "edges", "system")
_LEVEL_TO_GROUP = {"node": "atoms", "atoms": "atoms", "edge": "edges", "edges": "edges", "system": "system",
                   "graph": "system"}


class LevelSchema:
    """Attribute name → storage group (``atoms`` / ``edges`` / ``system``)."""

    def __init__(self, mapping: Mapping[str, str] | None = None) -> None:
        self._map: dict[str, str] = {}
        for k in _NODE_DEFAULT:
            self._map[k] = "atoms"
        for k in _EDGE_DEFAULT:
            self._map[k] = "edges"
        for k in _SYSTEM_DEFAULT:
            self._map[k] = "system"
        if mapping:
            for k, g in mapping.items():
                self.register(k, g)

    def register(self, key: str, level: str) -> None:
        if level not in _LEVEL_TO_GROUP:
            raise ValueError(f"unknown level {level!r}; expected node/edge/system")
        self._map[key] = _LEVEL_TO_GROUP[level]

    def group_of(self, key: str) -> str | None:
        return self._map.get(key)

    def copy(self) -> "LevelSchema":
        s = LevelSchema()
        s._map = dict(self._map)
        return s

    def as_dict(self) -> dict[str, str]:
        return dict(self._map)


def expand_segments(ptr: torch.Tensor, seg_idx: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Element indices of the segments ``seg_idx`` (in that order) and their lengths.

    ``ptr`` is the exclusive prefix of segment lengths (``[S+1]``).  Counterpart of the
    reference's ``_expand_segments_kernel`` (``data/level_storage.py:398-424``).
    """
    starts = ptr[seg_idx.long()].long()
    lens = (ptr[seg_idx.long() + 1] - ptr[seg_idx.long()]).long()
    return _buf.expand_segments(starts, lens), lens


class BaseLevelStorage:
    """Shared dictionary plumbing of the two storage kinds."""

    data: dict[str, torch.Tensor]

    def keys(self) -> Iterable[str]:
        return self.data.keys()

    def __contains__(self, key: str) -> bool:
        return key in self.data

    def __iter__(self) -> Iterator[str]:
        return iter(self.data)

    def __len__(self) -> int:
        return len(self.data)

    def __delitem__(self, key: str) -> None:
        del self.data[key]

    @property
    def device(self) -> torch.device | None:
        for v in self.data.values():
            return v.device
        return None


class UniformLevelStorage(BaseLevelStorage):
    """Rows indexed by system; ``num_valid`` rows are live, the rest is spare capacity."""

    def __init__(self, data: Mapping[str, torch.Tensor] | None = None, num_valid: int | None = None,
                 capacity: int | None = None) -> None:
        self.data = dict(data or {})
        cap = capacity if capacity is not None else (next(iter(self.data.values())).shape[0] if self.data else 0)
        self.capacity = int(cap)
        self.num_valid = int(self.capacity if num_valid is None else num_valid)

    def __getitem__(self, key: str) -> torch.Tensor:
        return self.data[key][: self.num_valid]

    def __setitem__(self, key: str, value: torch.Tensor) -> None:
        if key in self.data and self.data[key].shape[0] == self.capacity and value.shape[0] == self.num_valid \
                and self.capacity != self.num_valid:
            self.data[key][: self.num_valid] = value
            return
        if not self.data:
            self.capacity = value.shape[0]
            self.num_valid = value.shape[0]
        elif value.shape[0] != self.num_valid and value.shape[0] != self.capacity:
            raise ValueError(f"{key}: expected {self.num_valid} rows, got {value.shape[0]}")
        if value.shape[0] == self.num_valid and self.capacity != self.num_valid:
            full = value.new_zeros((self.capacity,) + tuple(value.shape[1:]))
            full[: self.num_valid] = value
            value = full
        self.data[key] = value

    def select(self, idx: torch.Tensor) -> "UniformLevelStorage":
        return UniformLevelStorage({k: v[: self.num_valid][idx] for k, v in self.data.items()},
                                   capacity=int(idx.numel()))

    def clone(self) -> "UniformLevelStorage":
        return UniformLevelStorage({k: v.clone() for k, v in self.data.items()}, self.num_valid, self.capacity)

    def to(self, *a: Any, **k: Any) -> "UniformLevelStorage":
        return UniformLevelStorage({n: v.to(*a, **k) for n, v in self.data.items()}, self.num_valid, self.capacity)

    def apply(self, fn: Any) -> "UniformLevelStorage":
        return UniformLevelStorage({n: fn(v) for n, v in self.data.items()}, self.num_valid, self.capacity)

    @staticmethod
    def concatenate(parts: list["UniformLevelStorage"]) -> "UniformLevelStorage":
        keys = [k for k in parts[0].data if all(k in p.data for p in parts)]
        return UniformLevelStorage({k: torch.cat([p[k] for p in parts], dim=0) for k in keys})

    def zero(self) -> None:
        for v in self.data.values():
            v.zero_()
        self.num_valid = 0

    # ---- fixed-capacity buffer operations ---------------------------------
    def free_rows(self) -> int:
        return self.capacity - self.num_valid

    def put(self, src: "UniformLevelStorage", take: torch.Tensor) -> None:
        """Append rows ``take`` (int64 indices into ``src``) after the live rows."""
        n = int(take.numel())
        if n == 0:
            return
        if n > self.free_rows():
            raise ValueError("UniformLevelStorage.put: not enough free rows")
        dst_rows = torch.arange(self.num_valid, self.num_valid + n, device=take.device)
        for k, dst in self.data.items():
            if k in src.data:
                _buf.copy_rows(src.data[k], take, dst, dst_rows)
        self.num_valid += n

    def defrag(self, keep: torch.Tensor) -> None:
        """Keep rows ``keep`` (sorted int64 indices of live rows); close the gaps in place."""
        n = int(keep.numel())
        dst_rows = torch.arange(n, device=keep.device)
        for k, v in self.data.items():
            _buf.compact_rows(v, keep, dst_rows, self.num_valid)
        self.num_valid = n


class SegmentedLevelStorage(BaseLevelStorage):
    """Concatenated variable-length segments (one per system) with CSR bookkeeping."""

    def __init__(self, data: Mapping[str, torch.Tensor] | None = None, lengths: torch.Tensor | None = None,
                 num_segments: int | None = None, num_elements: int | None = None,
                 segment_capacity: int | None = None, element_capacity: int | None = None,
                 device: torch.device | str | None = None) -> None:
        self.data = dict(data or {})
        dev = device if device is not None else (self.device or "cpu")
        if lengths is None:
            lengths = torch.zeros(0, dtype=torch.int32, device=dev)
        self.lengths = lengths.to(torch.int32)  # [segment_capacity]; zero beyond num_segments
        self.segment_capacity = int(segment_capacity if segment_capacity is not None else self.lengths.numel())
        self.num_segments = int(self.lengths.numel() if num_segments is None else num_segments)
        ecap = element_capacity
        if ecap is None:
            ecap = next(iter(self.data.values())).shape[0] if self.data else int(self.lengths.sum())
        self.element_capacity = int(ecap)
        self.num_elements = int(num_elements if num_elements is not None else
                                (self.lengths[: self.num_segments].sum().item() if self.num_segments else 0))
        self._ptr: torch.Tensor | None = None
        self._idx: torch.Tensor | None = None

    # ---- lazily derived CSR views -------------------------------------------
    def _invalidate(self) -> None:
        self._ptr = None
        self._idx = None

    @property
    def batch_ptr(self) -> torch.Tensor:
        if self._ptr is None:
            ptr = torch.zeros(self.num_segments + 1, dtype=torch.int32, device=self.lengths.device)
            if self.num_segments:
                torch.cumsum(self.lengths[: self.num_segments], 0, out=ptr[1:])
            self._ptr = ptr
        return self._ptr

    @property
    def batch_idx(self) -> torch.Tensor:
        if self._idx is None:
            seg = torch.arange(self.num_segments, dtype=torch.int32, device=self.lengths.device)
            self._idx = torch.repeat_interleave(seg, self.lengths[: self.num_segments].long(),
                                                output_size=self.num_elements)
        return self._idx

    @property
    def segment_lengths(self) -> torch.Tensor:
        return self.lengths[: self.num_segments]

    def __getitem__(self, key: str) -> torch.Tensor:
        return self.data[key][: self.num_elements]

    def __setitem__(self, key: str, value: torch.Tensor) -> None:
        if key in self.data and self.element_capacity != self.num_elements \
                and value.shape[0] == self.num_elements:
            self.data[key][: self.num_elements] = value
            return
        if self.data or self.num_segments:
            if value.shape[0] not in (self.num_elements, self.element_capacity):
                raise ValueError(f"{key}: expected {self.num_elements} rows, got {value.shape[0]}")
        if value.shape[0] == self.num_elements and self.element_capacity != self.num_elements:
            full = value.new_zeros((self.element_capacity,) + tuple(value.shape[1:]))
            full[: self.num_elements] = value
            value = full
        self.data[key] = value

    def select(self, seg_idx: torch.Tensor) -> tuple["SegmentedLevelStorage", torch.Tensor]:
        """New tight storage holding segments ``seg_idx``; also returns the gathered element indices."""
        elem, lens = expand_segments(self.batch_ptr, seg_idx)
        out = SegmentedLevelStorage({k: v[elem] for k, v in self.data.items()}, lens.to(torch.int32),
                                    num_elements=int(elem.numel()), device=self.lengths.device)
        return out, elem

    def clone(self) -> "SegmentedLevelStorage":
        return self._like({k: v.clone() for k, v in self.data.items()}, self.lengths.clone())

    def _like(self, data: dict[str, torch.Tensor], lengths: torch.Tensor) -> "SegmentedLevelStorage":
        return SegmentedLevelStorage(data, lengths, self.num_segments, self.num_elements, self.segment_capacity,
                                     self.element_capacity, device=lengths.device)

    def to(self, *a: Any, **k: Any) -> "SegmentedLevelStorage":
        kk = {x: y for x, y in k.items() if x != "dtype"}
        return self._like({n: v.to(*a, **k) for n, v in self.data.items()}, self.lengths.to(*a, **kk))

    def apply(self, fn: Any) -> "SegmentedLevelStorage":
        return self._like({n: fn(v) for n, v in self.data.items()}, fn(self.lengths))

    @staticmethod
    def concatenate(parts: list["SegmentedLevelStorage"]) -> "SegmentedLevelStorage":
        keys = [k for k in parts[0].data if all(k in p.data for p in parts)]
        data = {k: torch.cat([p[k] for p in parts], dim=0) for k in keys}
        lens = torch.cat([p.segment_lengths for p in parts])
        return SegmentedLevelStorage(data, lens, num_elements=sum(p.num_elements for p in parts),
                                     device=lens.device)

    def zero(self) -> None:
        for v in self.data.values():
            v.zero_()
        self.lengths.zero_()
        self.num_segments = 0
        self.num_elements = 0
        self._invalidate()

    # ---- fixed-capacity buffer operations ---------------------------------
    def free_segments(self) -> int:
        return self.segment_capacity - self.num_segments

    def free_elements(self) -> int:
        return self.element_capacity - self.num_elements

    def put(self, src: "SegmentedLevelStorage", take: torch.Tensor) -> torch.Tensor:
        """Append segments ``take`` of ``src``; returns per-copied-element destination rows."""
        n = int(take.numel())
        if n == 0:
            return take.new_zeros(0)
        elem, lens = expand_segments(src.batch_ptr, take)
        m = int(elem.numel())
        if n > self.free_segments() or m > self.free_elements():
            raise ValueError("SegmentedLevelStorage.put: not enough capacity")
        dst_rows = torch.arange(self.num_elements, self.num_elements + m, device=take.device)
        for k, dst in self.data.items():
            if k in src.data:
                _buf.copy_rows(src.data[k], elem, dst, dst_rows)
        self.lengths[self.num_segments: self.num_segments + n] = lens.to(torch.int32)
        self.num_segments += n
        self.num_elements += m
        self._invalidate()
        return dst_rows

    def defrag(self, keep: torch.Tensor) -> torch.Tensor:
        """Keep segments ``keep`` (sorted); compact in place.  Returns old element index per kept row."""
        elem, lens = expand_segments(self.batch_ptr, keep)
        m = int(elem.numel())
        dst_rows = torch.arange(m, device=elem.device)
        for k, v in self.data.items():
            _buf.compact_rows(v, elem, dst_rows, self.num_elements)
        n = int(keep.numel())
        new_len = torch.zeros_like(self.lengths)
        new_len[:n] = lens.to(torch.int32)
        self.lengths = new_len
        self.num_segments = n
        self.num_elements = m
        self._invalidate()
        return elem


class MultiLevelStorage:
    """Router over the ``atoms`` / ``edges`` / ``system`` groups."""

    def __init__(self, atoms: SegmentedLevelStorage | None = None, edges: SegmentedLevelStorage | None = None,
                 system: UniformLevelStorage | None = None, schema: LevelSchema | None = None) -> None:
        self.groups: dict[str, BaseLevelStorage | None] = {"atoms": atoms, "edges": edges, "system": system}
        self.schema = schema or LevelSchema()

    @property
    def atoms(self) -> SegmentedLevelStorage | None:
        return self.groups["atoms"]  # type: ignore[return-value]

    @property
    def edges(self) -> SegmentedLevelStorage | None:
        return self.groups["edges"]  # type: ignore[return-value]

    @property
    def system(self) -> UniformLevelStorage | None:
        return self.groups["system"]  # type: ignore[return-value]

    def group_of(self, key: str) -> str | None:
        for name, g in self.groups.items():
            if g is not None and key in g:
                return name
        return self.schema.group_of(key)

    def __contains__(self, key: str) -> bool:
        return any(g is not None and key in g for g in self.groups.values())

    def __getitem__(self, key: str) -> torch.Tensor:
        for g in self.groups.values():
            if g is not None and key in g:
                return g[key]
        raise KeyError(key)

    def __setitem__(self, key: str, value: torch.Tensor) -> None:
        name = self.group_of(key)
        if name is None:
            raise KeyError(f"'{key}' has no known level; register it with add_key(level=...) first")
        g = self.groups[name]
        if g is None:
            raise KeyError(f"group '{name}' does not exist in this batch")
        g[key] = value

    def __delitem__(self, key: str) -> None:
        for g in self.groups.values():
            if g is not None and key in g:
                del g[key]
                return
        raise KeyError(key)

    def keys(self) -> list[str]:
        out: list[str] = []
        for g in self.groups.values():
            if g is not None:
                out.extend(sorted(g.keys()))
        return out

    def items(self) -> Iterator[tuple[str, torch.Tensor]]:
        for k in self.keys():
            yield k, self[k]

    def map_groups(self, fn: Any) -> "MultiLevelStorage":
        return MultiLevelStorage(*(None if g is None else fn(g) for g in self.groups.values()),
                                 schema=self.schema.copy())
