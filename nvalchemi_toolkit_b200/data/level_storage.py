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


def _as(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    src = src if src.dtype == dst.dtype else src.to(dst.dtype)
    return src if src.is_contiguous() else src.contiguous()


def _compact_through_scratch(ops: Any, v: torch.Tensor, old_ptr: torch.Tensor, plan: torch.Tensor, n_rows: int) -> None:
    """In-place compaction of the first ``n_rows`` rows of ``v``: kept segments go to a zeroed scratch copy and back, so
    vacated rows end up zero and overlapping moves cannot clobber one another."""
    if n_rows == 0:
        return
    head = v[:n_rows]
    tmp = torch.zeros_like(head)
    ops.segmented_copy_planned(head, old_ptr, plan, tmp)
    head.copy_(tmp)


class DeviceCounts:
    """Row / segment counts that a device-side put or defrag produced, read back to the host only when someone asks.

    ``tensor`` is a small int32 device vector; :meth:`host` copies it once (the only synchronisation of a masked put) and
    caches the integers.  The storages of one batch share one instance, so the three levels resolve with one copy."""

    def __init__(self, tensor: torch.Tensor) -> None:
        self.tensor, self._host = tensor, None

    def host(self) -> list[int]:
        if self._host is None:
            self._host = [int(x) for x in self.tensor.tolist()]
        return self._host


def _buffer_ops() -> Any:
    """The native masked put / defrag operators, or ``None`` when the library is not built (pure-torch fallback)."""
    from nvalchemi_toolkit_b200.ops import _native

    return torch.ops.nvalchemi if _native.available() and hasattr(torch.ops.nvalchemi, "segmented_put_plan") else None


class UniformLevelStorage(BaseLevelStorage):
    """Rows indexed by system; ``num_valid`` rows are live, the rest is spare capacity."""

    def __init__(self, data: Mapping[str, torch.Tensor] | None = None, num_valid: int | None = None,
                 capacity: int | None = None) -> None:
        self.data = dict(data or {})
        cap = capacity if capacity is not None else (next(iter(self.data.values())).shape[0] if self.data else 0)
        self.capacity = int(cap)
        self._pending: tuple[DeviceCounts, int] | None = None
        self._count_dev: torch.Tensor | None = None
        self.num_valid = int(self.capacity if num_valid is None else num_valid)

    @property
    def num_valid(self) -> int:
        if self._pending is not None:
            counts, i = self._pending
            self._n_valid, self._pending = counts.host()[i], None
        return self._n_valid

    @num_valid.setter
    def num_valid(self, n: int) -> None:
        self._n_valid, self._pending, self._count_dev = int(n), None, None

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

    # ---- device-planned variants (no index lists, no counts on the host) ---------------------------------------
    def _unit_ptr(self, n: int, device: torch.device) -> torch.Tensor:
        """``[0, 1, ..., n]``: a uniform level is a segmented one whose segments all have one row."""
        return torch.arange(n + 1, dtype=torch.int32, device=device)

    def device_count(self, device: torch.device) -> torch.Tensor:
        if self._count_dev is None:
            self._count_dev = torch.tensor([self._n_valid], dtype=torch.int32).to(device, non_blocking=True)
        return self._count_dev

    def put_masked(self, ops: Any, src: "UniformLevelStorage", take: torch.Tensor, n_src: int) -> None:
        """Append the rows of ``src`` flagged in ``take`` (bool, device) behind the live rows; the new row count stays on
        the device until :attr:`num_valid` is read."""
        dev = take.device
        count = self.device_count(dev)
        went = torch.empty(n_src, dtype=torch.bool, device=dev)
        sp = self._unit_ptr(n_src, dev)
        plan = ops.segmented_put_plan(sp, take, self._unit_ptr(self.capacity, dev), count, self.capacity, went, True)
        for k, dst in self.data.items():
            if k in src.data:
                ops.segmented_copy_planned(_as(src.data[k], dst), sp, plan, dst)

    def defrag_masked(self, ops: Any, removed: torch.Tensor, n_live: int) -> None:
        dev = removed.device
        count = self.device_count(dev)
        ptr = self._unit_ptr(n_live, dev)
        plan, old = ops.segmented_defrag_plan(ptr, removed, count)
        for v in self.data.values():
            _compact_through_scratch(ops, v, old, plan, n_live)

    def set_pending(self, counts: DeviceCounts, index: int) -> None:
        self._pending = (counts, index)  # the device counter stays valid: only the host copy is stale

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
        self._pending: tuple[DeviceCounts, int, int] | None = None
        self._csr_dev: tuple[torch.Tensor, torch.Tensor] | None = None
        self.num_segments = int(self.lengths.numel() if num_segments is None else num_segments)
        ecap = element_capacity
        if ecap is None:
            ecap = next(iter(self.data.values())).shape[0] if self.data else int(self.lengths.sum())
        self.element_capacity = int(ecap)
        self.num_elements = int(num_elements if num_elements is not None else
                                (self.lengths[: self.num_segments].sum().item() if self.num_segments else 0))
        self._ptr: torch.Tensor | None = None
        self._idx: torch.Tensor | None = None

    # ---- counts: host integers, or still on the device after a masked put / defrag --------------------------------
    def _resolve(self) -> None:
        if self._pending is not None:
            counts, i_seg, i_elem = self._pending
            host = counts.host()
            self._n_seg, self._n_elem, self._pending = host[i_seg], host[i_elem], None

    @property
    def num_segments(self) -> int:
        self._resolve()
        return self._n_seg

    @num_segments.setter
    def num_segments(self, n: int) -> None:
        self._resolve()
        self._n_seg, self._csr_dev = int(n), None

    @property
    def num_elements(self) -> int:
        self._resolve()
        return self._n_elem

    @num_elements.setter
    def num_elements(self, n: int) -> None:
        self._resolve()
        self._n_elem, self._csr_dev = int(n), None

    # ---- lazily derived CSR views -------------------------------------------
    def _invalidate(self) -> None:
        self._ptr = None
        self._idx = None
        self._csr_dev = None

    def device_csr(self) -> tuple[torch.Tensor, torch.Tensor]:
        """``(ptr, count)`` on the device: ``ptr`` has ``segment_capacity + 1`` entries whose first ``count + 1`` are the
        row offsets of the live segments.  The masked put / defrag operators read and update both in place."""
        if self._csr_dev is None:
            dev = self.lengths.device
            ptr = torch.zeros(self.segment_capacity + 1, dtype=torch.int32, device=dev)
            n = min(int(self.lengths.numel()), self.segment_capacity)
            if n:
                torch.cumsum(self.lengths[:n], 0, out=ptr[1: n + 1])  # lengths are zero behind the live segments
                if n < self.segment_capacity:
                    ptr[n + 1:] = ptr[n]
            count = torch.tensor([self._n_seg], dtype=torch.int32).to(dev, non_blocking=True)
            self._csr_dev = (ptr, count)
        return self._csr_dev

    def _adopt_device_csr(self, counts: DeviceCounts, i_seg: int, i_elem: int) -> None:
        """After a device-side update of ``(ptr, count)``: refresh ``lengths`` from them (on the device) and leave the host
        counts pending."""
        ptr, count = self._csr_dev
        cap = self.segment_capacity
        live = torch.arange(cap, device=ptr.device) < count
        lengths = torch.where(live, ptr[1:] - ptr[:-1], torch.zeros((), dtype=torch.int32, device=ptr.device))
        if self.lengths.numel() == cap:
            self.lengths.copy_(lengths)
        else:
            self.lengths = lengths
        self._ptr = self._idx = None
        self._pending = (counts, i_seg, i_elem)

    def put_masked(self, ops: Any, src_ptr: torch.Tensor, take: torch.Tensor, went: torch.Tensor, src_data: Mapping[str, torch.Tensor],
                   commit: bool = True) -> torch.Tensor:
        """Append the source segments flagged in ``take`` that fit (``went`` receives which); with ``commit=False`` only
        the fit mask is computed.  Returns the plan (first destination row per source segment, or -1)."""
        ptr, count = self.device_csr()
        plan = ops.segmented_put_plan(src_ptr, take, ptr, count, self.element_capacity, went, commit)
        if commit:
            for k, dst in self.data.items():
                if k in src_data:
                    ops.segmented_copy_planned(_as(src_data[k], dst), src_ptr, plan, dst)
        return plan

    def defrag_masked(self, ops: Any, removed: torch.Tensor, n_live: int, n_rows: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Drop the live segments flagged in ``removed``; returns ``(plan, old_ptr)``."""
        ptr, count = self.device_csr()
        plan, old = ops.segmented_defrag_plan(ptr[: n_live + 1], removed, count)
        for v in self.data.values():
            _compact_through_scratch(ops, v, old, plan, n_rows)
        return plan, old

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
