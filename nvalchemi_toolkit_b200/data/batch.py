# SPDX-License-Identifier: Apache-2.0
"""``Batch``: many systems concatenated into three columnar groups.

Public behaviour follows the reference's ``nvalchemi/data/batch.py:182-1839``:
construction from ``AtomicData`` lists or raw dictionaries, pre-allocated
fixed-capacity buffers (``empty`` + ``put`` / ``defrag`` / ``trim``), graph-level
``index_select``, ``append``, ``add_key``, device moves, and a point-to-point wire
protocol (header ``int64[3]`` → segment lengths → one message per field in
sorted key order).  ``neighbor_list`` is the only index-valued key: its entries
are offset by the node offset of their graph on concatenation
(``data/batch.py:60`` in the reference).
"""
from __future__ import annotations

from typing import Any, Iterator, Sequence

import numpy as np
import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData, DataMixin
from nvalchemi_toolkit_b200.data.level_storage import (
    DeviceCounts, LevelSchema, MultiLevelStorage, SegmentedLevelStorage, UniformLevelStorage, _buffer_ops,
)

_INDEX_KEYS = frozenset({"neighbor_list"})
_OWN_ATTRS = frozenset({"_storage", "_data_class", "device", "keys"})


def _group_items(data: AtomicData) -> dict[str, dict[str, torch.Tensor]]:
    return {"atoms": data.node_properties, "edges": data.edge_properties, "system": data.system_properties}


class Batch(DataMixin):
    """Graph-aware batch over a :class:`MultiLevelStorage`."""

    def __init__(self, *, device: torch.device | str, storage: MultiLevelStorage | None = None,
                 keys: dict[str, set[str]] | None = None) -> None:
        object.__setattr__(self, "_storage", storage if storage is not None else MultiLevelStorage())
        object.__setattr__(self, "_data_class", AtomicData)
        object.__setattr__(self, "device", torch.device(device))
        object.__setattr__(self, "keys", keys)

    # ------------------------------------------------------------ attribute IO
    def __setattr__(self, name: str, value: Any) -> None:
        if name in _OWN_ATTRS or not isinstance(value, torch.Tensor):
            object.__setattr__(self, name, value)
        else:
            self._storage[name] = value

    def __getattr__(self, name: str) -> Any:
        if name.startswith("__"):
            raise AttributeError(name)
        storage = object.__getattribute__(self, "_storage")
        if name in storage:
            return storage[name]
        if storage.schema.group_of(name) is not None or name in AtomicData.model_fields:
            return None
        raise AttributeError(f"Batch has no attribute {name!r}")

    def __getitem__(self, key: Any) -> Any:
        if isinstance(key, str):
            if key in self._storage:
                return self._storage[key]
            if key in ("batch_idx", "batch_ptr", "edge_ptr"):
                return getattr(self, key)
            raise KeyError(key)
        if isinstance(key, (int, np.integer)):
            return self.get_data(int(key))
        return self.index_select(key)

    def __setitem__(self, key: str, value: Any) -> None:
        setattr(self, key, value)

    def __delitem__(self, key: str) -> None:
        del self._storage[key]

    def __contains__(self, key: str) -> bool:
        return key in self._storage

    def __len__(self) -> int:
        return self.num_graphs

    def __iter__(self) -> Iterator[tuple[str, torch.Tensor]]:
        return iter(self._storage.items())

    def __repr__(self) -> str:
        return (f"Batch(num_graphs={self.num_graphs}, num_nodes={self.num_nodes}, num_edges={self.num_edges}, "
                f"device={self.device}, keys={self._storage.keys()})")

    # -------------------------------------------------------------- properties
    @property
    def _atoms_group(self) -> SegmentedLevelStorage | None:
        return self._storage.atoms

    @property
    def _edges_group(self) -> SegmentedLevelStorage | None:
        return self._storage.edges

    @property
    def _system_group(self) -> UniformLevelStorage | None:
        return self._storage.system

    @property
    def num_graphs(self) -> int:
        if self._atoms_group is not None:
            return self._atoms_group.num_segments
        return self._system_group.num_valid if self._system_group is not None else 0

    batch_size = num_graphs

    @property
    def num_nodes(self) -> int:
        return self._atoms_group.num_elements if self._atoms_group is not None else 0

    @property
    def num_edges(self) -> int:
        return self._edges_group.num_elements if self._edges_group is not None else 0

    @property
    def system_capacity(self) -> int:
        if self._system_group is not None:
            return self._system_group.capacity
        return self._atoms_group.segment_capacity if self._atoms_group is not None else 0

    @property
    def batch_idx(self) -> torch.Tensor:
        return self._atoms_group.batch_idx

    @property
    def batch_ptr(self) -> torch.Tensor:
        return self._atoms_group.batch_ptr

    @property
    def edge_ptr(self) -> torch.Tensor:
        if self._edges_group is None:
            return torch.zeros(self.num_graphs + 1, dtype=torch.int32, device=self.device)
        return self._edges_group.batch_ptr

    @property
    def num_nodes_per_graph(self) -> torch.Tensor:
        return self._atoms_group.segment_lengths

    @property
    def num_edges_per_graph(self) -> torch.Tensor:
        if self._edges_group is None:
            return torch.zeros(self.num_graphs, dtype=torch.int32, device=self.device)
        return self._edges_group.segment_lengths

    @property
    def num_nodes_list(self) -> list[int]:
        return self.num_nodes_per_graph.tolist()

    @property
    def num_edges_list(self) -> list[int]:
        return self.num_edges_per_graph.tolist()

    @property
    def max_num_nodes(self) -> int:
        return int(self.num_nodes_per_graph.max()) if self.num_graphs else 0

    # ------------------------------------------------------------ construction
    @classmethod
    def _construct(cls, *, device: torch.device | str, keys: dict[str, set[str]] | None,
                   storage: MultiLevelStorage, data_class: type = AtomicData) -> "Batch":
        b = cls.__new__(cls)
        object.__setattr__(b, "_storage", storage)
        object.__setattr__(b, "_data_class", data_class)
        object.__setattr__(b, "device", torch.device(device))
        object.__setattr__(b, "keys", keys)
        return b

    @classmethod
    def from_data_list(cls, data_list: Sequence[AtomicData], device: torch.device | str | None = None,
                       exclude_keys: Sequence[str] | None = None) -> "Batch":
        if len(data_list) == 0:
            raise ValueError("from_data_list needs at least one AtomicData")
        dicts = []
        schema = LevelSchema()
        for d in data_list:
            g = _group_items(d)
            merged: dict[str, torch.Tensor] = {}
            for gname, items in g.items():
                for k, v in items.items():
                    schema.register(k, {"atoms": "node", "edges": "edge", "system": "system"}[gname])
                    merged[k] = v
            dicts.append(merged)
        return cls.from_raw_dicts(dicts, schema=schema, device=device, exclude_keys=exclude_keys,
                                  data_class=type(data_list[0]))

    @classmethod
    def from_raw_dicts(cls, dicts: Sequence[dict[str, torch.Tensor]], field_levels: dict[str, str] | None = None,
                       schema: LevelSchema | None = None, device: torch.device | str | None = None,
                       exclude_keys: Sequence[str] | None = None, data_class: type = AtomicData) -> "Batch":
        """Concatenate per-sample dictionaries without constructing ``AtomicData`` (no validation)."""
        schema = schema.copy() if schema is not None else LevelSchema()
        for k, lvl in (field_levels or {}).items():
            schema.register(k, lvl)
        exclude = set(exclude_keys or ())
        common = [k for k in dicts[0] if k not in exclude and isinstance(dicts[0][k], torch.Tensor)
                  and all(isinstance(d.get(k), torch.Tensor) for d in dicts)]
        common.sort()  # deterministic key order keeps collectives aligned across ranks
        dev = torch.device(device) if device is not None else dicts[0]["positions"].device
        n_nodes = torch.tensor([d["positions"].shape[0] for d in dicts], dtype=torch.int32)
        has_edges = "neighbor_list" in common
        n_edges = torch.tensor([d["neighbor_list"].shape[0] if has_edges else 0 for d in dicts], dtype=torch.int32)
        node_off = torch.cumsum(n_nodes, 0) - n_nodes
        groups: dict[str, dict[str, torch.Tensor]] = {"atoms": {}, "edges": {}, "system": {}}
        for k in common:
            g = schema.group_of(k)
            if g is None:
                continue
            if g == "edges" and not has_edges:
                continue
            parts = [d[k] for d in dicts]
            if k in _INDEX_KEYS:
                parts = [p + int(o) for p, o in zip(parts, node_off.tolist())]
            if g == "system":
                parts = [p if p.dim() >= 1 and p.shape[0] == 1 else p.unsqueeze(0) for p in parts]
            groups[g][k] = torch.cat(parts, dim=0).to(dev)
        atoms = SegmentedLevelStorage(groups["atoms"], n_nodes.to(dev), num_elements=int(n_nodes.sum()), device=dev)
        edges = SegmentedLevelStorage(groups["edges"], n_edges.to(dev), num_elements=int(n_edges.sum()),
                                      device=dev) if has_edges else None
        system = UniformLevelStorage(groups["system"], capacity=len(dicts))
        storage = MultiLevelStorage(atoms, edges, system, schema)
        keys = {"node": set(groups["atoms"]), "edge": set(groups["edges"]), "system": set(groups["system"])}
        return cls._construct(device=dev, keys=keys, storage=storage, data_class=data_class)

    @classmethod
    def empty(cls, *, num_systems: int, num_nodes: int, num_edges: int,
              template: "AtomicData | Batch | None" = None, device: torch.device | str = "cpu",
              attr_map: LevelSchema | None = None) -> "Batch":
        """Pre-allocated buffer with zero graphs; fill it with :meth:`put`."""
        dev = torch.device(device)
        if template is None:
            template = AtomicData(atomic_numbers=torch.ones(1, dtype=torch.long), positions=torch.zeros(1, 3),
                                  energy=torch.zeros(1, 1))
        if isinstance(template, AtomicData):
            template = cls.from_data_list([template])
        schema = (attr_map or template._storage.schema).copy()

        def alloc(g: Any, rows: int) -> dict[str, torch.Tensor]:
            return {} if g is None else {k: torch.zeros((rows,) + tuple(v.shape[1:]), dtype=v.dtype, device=dev)
                                         for k, v in g.data.items()}

        atoms = SegmentedLevelStorage(alloc(template._atoms_group, num_nodes),
                                      torch.zeros(num_systems, dtype=torch.int32, device=dev), num_segments=0,
                                      num_elements=0, segment_capacity=num_systems, element_capacity=num_nodes,
                                      device=dev)
        edges = None
        if template._edges_group is not None and num_edges > 0:
            edges = SegmentedLevelStorage(alloc(template._edges_group, num_edges),
                                          torch.zeros(num_systems, dtype=torch.int32, device=dev), num_segments=0,
                                          num_elements=0, segment_capacity=num_systems, element_capacity=num_edges,
                                          device=dev)
        system = UniformLevelStorage(alloc(template._system_group, num_systems), num_valid=0, capacity=num_systems)
        keys = {k: set(v) for k, v in (template.keys or {}).items()}
        return cls._construct(device=dev, keys=keys, storage=MultiLevelStorage(atoms, edges, system, schema),
                              data_class=template._data_class)

    @classmethod
    def empty_like(cls, other: "Batch", num_systems: int | None = None, num_nodes: int | None = None,
                   num_edges: int | None = None, device: torch.device | str | None = None) -> "Batch":
        return cls.empty(num_systems=num_systems or max(other.system_capacity, 1),
                         num_nodes=num_nodes or max(other.num_nodes, 1),
                         num_edges=num_edges if num_edges is not None else other.num_edges,
                         template=other, device=device or other.device)

    def zero(self) -> None:
        """Reset a buffer to zero graphs (capacity retained)."""
        for g in self._storage.groups.values():
            if g is not None:
                g.zero()

    # ---------------------------------------------------------------- queries
    def get_data(self, idx: int) -> AtomicData:
        n = self.num_graphs
        if idx < 0:
            idx += n
        if not 0 <= idx < n:
            raise IndexError(f"graph index {idx} out of range for {n} graphs")
        sub = self.index_select([idx])
        kw: dict[str, Any] = {k: v for k, v in sub._storage.items()}
        kw.pop("status", None) if "status" not in self._storage else None
        data = self._data_class.model_construct(**kw)
        data.model_post_init(None)
        for k in kw:
            g = sub._storage.group_of(k)
            {"atoms": data.__node_keys__, "edges": data.__edge_keys__, "system": data.__system_keys__}[g].add(k)
        return data

    def to_data_list(self) -> list[AtomicData]:
        return [self.get_data(i) for i in range(self.num_graphs)]

    def _normalize_index(self, idx: Any) -> torch.Tensor:
        n = self.num_graphs
        if isinstance(idx, (int, np.integer)):
            idx = [int(idx)]
        if isinstance(idx, slice):
            idx = list(range(*idx.indices(n)))
        t = torch.as_tensor(idx, device=self.device) if not isinstance(idx, torch.Tensor) else idx.to(self.device)
        if t.dtype == torch.bool:
            if t.numel() != n:
                raise IndexError("boolean graph mask has the wrong length")
            t = torch.nonzero(t).squeeze(1)
        t = t.long().reshape(-1)
        return torch.where(t < 0, t + n, t)

    def index_select(self, idx: Any) -> "Batch":
        """Subset of graphs (tight storage) selected by int / slice / list / tensor / bool mask."""
        sel = self._normalize_index(idx)
        atoms, _ = self._atoms_group.select(sel)
        edges = None
        if self._edges_group is not None:
            edges, _ = self._edges_group.select(sel)
            if "neighbor_list" in edges.data and edges.num_elements:
                old_off = self.batch_ptr[sel].long()
                new_off = (atoms.batch_ptr[:-1]).long()
                delta = torch.repeat_interleave(new_off - old_off, edges.segment_lengths.long(),
                                                output_size=edges.num_elements)
                edges.data["neighbor_list"] = edges.data["neighbor_list"] + delta[:, None]
        system = self._system_group.select(sel) if self._system_group is not None else None
        storage = MultiLevelStorage(atoms, edges, system, self._storage.schema.copy())
        keys = None if self.keys is None else {k: set(v) for k, v in self.keys.items()}
        return Batch._construct(device=self.device, keys=keys, storage=storage, data_class=self._data_class)

    # ------------------------------------------------------- buffer operations
    def put(self, src_batch: "Batch", mask: torch.Tensor, *, copied_mask: torch.Tensor | None = None,
            dest_mask: torch.Tensor | None = None) -> None:
        """Copy the graphs of ``src_batch`` flagged in ``mask`` into this buffer, as many as fit.

        Graphs are considered in index order; one is copied only if it fits in the system,
        atom and edge capacities together.  ``copied_mask`` (or ``src_batch._copied_mask``)
        receives the mask of graphs actually copied, for a following :meth:`defrag`.
        """
        mask = mask.to(self.device).bool().reshape(-1)[: src_batch.num_graphs]
        ops = _buffer_ops()
        if ops is not None and self._atoms_group is not None and src_batch._atoms_group is not None:
            self._put_planned(ops, src_batch, mask.contiguous(), copied_mask)
            return
        cand = torch.nonzero(mask).squeeze(1)
        na = src_batch.num_nodes_per_graph.long()[cand]
        fits = torch.arange(1, cand.numel() + 1, device=self.device) <= (self.system_capacity - self.num_graphs)
        fits &= torch.cumsum(na, 0) <= self._atoms_group.free_elements()
        has_e = self._edges_group is not None and src_batch._edges_group is not None
        if has_e:
            ne = src_batch.num_edges_per_graph.long()[cand]
            fits &= torch.cumsum(ne, 0) <= self._edges_group.free_elements()
        take = cand[fits]
        node_base = self.num_nodes
        first_new_edge = self.num_edges
        self._atoms_group.put(src_batch._atoms_group, take)
        if has_e:
            self._edges_group.put(src_batch._edges_group, take)
            if "neighbor_list" in self._edges_group.data and take.numel():
                # re-base copied node indices: subtract source offset, add destination offset
                src_off = src_batch.batch_ptr[take].long()
                lens_a = src_batch.num_nodes_per_graph.long()[take]
                dst_off = node_base + torch.cumsum(lens_a, 0) - lens_a
                lens_e = src_batch.num_edges_per_graph.long()[take]
                delta = torch.repeat_interleave(dst_off - src_off, lens_e)
                nl = self._edges_group.data["neighbor_list"]
                nl[first_new_edge: first_new_edge + delta.numel()] += delta[:, None]
        elif self._edges_group is not None:
            n = int(take.numel())
            self._edges_group.num_segments += n
            self._edges_group._invalidate()
        if self._system_group is not None and src_batch._system_group is not None:
            self._system_group.put(src_batch._system_group, take)
        done = torch.zeros(src_batch.num_graphs, dtype=torch.bool, device=self.device)
        done[take] = True
        if copied_mask is not None:
            copied_mask[: done.numel()] = done
        else:
            object.__setattr__(src_batch, "_copied_mask", done)

    # ---- device-planned put / defrag: masks in, masks out, counts stay on the device ---------------------------
    def _put_planned(self, ops: Any, src: "Batch", mask: torch.Tensor, copied_mask: torch.Tensor | None) -> None:
        """Masked put through the native planners (``segmented_put_plan`` / ``segmented_copy_planned``; the reference's
        ``put_masked_segmented`` / ``put_masked_per_system`` chain, ``nvalchemi/data/level_storage.py``): the fit over
        atoms, edges and systems, the slot assignment and every copy run on the device, and the new counts are read by
        the host only when ``num_graphs`` / ``num_nodes`` / ``num_edges`` are next asked for."""
        dev = self.device
        n_src = src.num_graphs
        a, e, sysg = self._atoms_group, self._edges_group, self._system_group
        sa, se = src._atoms_group, src._edges_group
        done = torch.zeros(max(n_src, 1), dtype=torch.bool, device=dev)[:n_src]
        if n_src == 0:
            self._publish_copied(src, done, copied_mask)
            return
        a_ptr = sa.batch_ptr
        zero_ptr = torch.zeros(n_src + 1, dtype=torch.int32, device=dev)
        e_ptr = se.batch_ptr if (e is not None and se is not None) else zero_ptr
        fit = torch.empty_like(done)
        a.put_masked(ops, a_ptr, mask, fit, {}, commit=False)              # fits the atom rows and the system slots
        if e is not None:
            fit_e = torch.empty_like(done)
            e.put_masked(ops, e_ptr, fit, fit_e, {}, commit=False)        # ... and the edge rows
            fit = fit_e  # a subset of a fitting set still fits the atoms: offsets only shrink
        plan_a = a.put_masked(ops, a_ptr, fit, done, {k: v for k, v in sa.data.items()})
        if e is not None:
            src_edges: dict[str, torch.Tensor] = dict(se.data) if se is not None else {}
            if "neighbor_list" in src_edges and "neighbor_list" in e.data and src.num_edges:
                # re-base node indices: minus the graph's source offset, plus its destination offset
                delta = (plan_a - a_ptr[:-1])[se.batch_idx.long()]
                nl = src_edges["neighbor_list"][: src.num_edges]
                src_edges["neighbor_list"] = nl + delta.to(nl.dtype)[:, None]
            went_e = torch.empty_like(done)
            e.put_masked(ops, e_ptr, fit, went_e, src_edges)
        if sysg is not None:
            sysg.put_masked(ops, src._system_group if src._system_group is not None else UniformLevelStorage({}, 0, 0), fit, n_src)
        self._adopt_counts()
        self._publish_copied(src, done, copied_mask)

    def _adopt_counts(self) -> None:
        a, e, sysg = self._atoms_group, self._edges_group, self._system_group
        ptr_a, count_a = a.device_csr()
        idx = count_a.long()
        parts = [count_a, ptr_a[idx]]
        if e is not None:
            ptr_e, count_e = e.device_csr()
            parts.append(ptr_e[count_e.long()])
        counts = DeviceCounts(torch.cat([p.reshape(1) for p in parts]))
        a._adopt_device_csr(counts, 0, 1)
        if e is not None:
            e._adopt_device_csr(counts, 0, 2)
        if sysg is not None:
            sysg.set_pending(counts, 0)

    @staticmethod
    def _publish_copied(src: "Batch", done: torch.Tensor, copied_mask: torch.Tensor | None) -> None:
        if copied_mask is not None:
            copied_mask[: done.numel()] = done
        else:
            object.__setattr__(src, "_copied_mask", done)

    def _defrag_planned(self, ops: Any, removed: torch.Tensor, n: int) -> None:
        a, e, sysg = self._atoms_group, self._edges_group, self._system_group
        n_nodes, n_edges = self.num_nodes, self.num_edges
        e_idx = e.batch_idx.long() if (e is not None and "neighbor_list" in e.data and n_edges) else None
        plan_a, old_a = a.defrag_masked(ops, removed, n, n_nodes)
        if e is not None:
            if e_idx is not None:
                delta = (plan_a - old_a[:-1])[e_idx]  # rows of dropped graphs get a meaningless shift and are dropped too
                nl = e.data["neighbor_list"]
                nl[:n_edges] += delta.to(nl.dtype)[:, None]
            e.defrag_masked(ops, removed, n, n_edges)
        if sysg is not None:
            sysg.defrag_masked(ops, removed, n)
        self._adopt_counts()

    def defrag(self, copied_mask: torch.Tensor | None = None) -> "Batch":
        """Remove the graphs flagged in ``copied_mask`` in place, keeping capacity."""
        if copied_mask is None:
            copied_mask = getattr(self, "_copied_mask", None)
            if copied_mask is None:
                return self
        n = self.num_graphs
        ops = _buffer_ops()
        if ops is not None and self._atoms_group is not None:
            self._defrag_planned(ops, copied_mask.to(self.device).bool().reshape(-1)[:n].contiguous(), n)
            object.__setattr__(self, "_copied_mask", None)
            return self
        keep = torch.nonzero(~copied_mask.to(self.device).bool()[:n]).squeeze(1)
        if keep.numel() == n:
            return self
        old_ptr = self.batch_ptr.long()
        self._atoms_group.defrag(keep)
        if self._edges_group is not None:
            nl_key = "neighbor_list" in self._edges_group.data
            old_e_lens = self._edges_group.segment_lengths.long()[keep]
            self._edges_group.defrag(keep)
            if nl_key and self._edges_group.num_elements:
                new_ptr = self.batch_ptr.long()
                delta = torch.repeat_interleave(new_ptr[:-1] - old_ptr[keep], old_e_lens,
                                                output_size=self._edges_group.num_elements)
                self._edges_group.data["neighbor_list"][: delta.numel()] += delta[:, None]
        if self._system_group is not None:
            self._system_group.defrag(keep)
        object.__setattr__(self, "_copied_mask", None)
        return self

    def trim(self, copied_mask: torch.Tensor | None = None) -> "Batch | None":
        """New tight batch without the flagged graphs; ``None`` when nothing remains."""
        if copied_mask is None:
            copied_mask = getattr(self, "_copied_mask", None)
        n = self.num_graphs
        if copied_mask is None:
            keep = torch.arange(n, device=self.device)
        else:
            keep = torch.nonzero(~copied_mask.to(self.device).bool()[:n]).squeeze(1)
        if keep.numel() == 0:
            return None
        return self.index_select(keep)

    # ---------------------------------------------------------------- growing
    def append(self, other: "Batch") -> None:
        """Concatenate ``other`` after this batch (in place; keys missing on either side are dropped)."""
        node_off = self.num_nodes
        mine, theirs = self._tight(), other._tight()
        atoms = SegmentedLevelStorage.concatenate([mine._atoms_group, theirs._atoms_group])
        edges = None
        if mine._edges_group is not None and theirs._edges_group is not None:
            te = theirs._edges_group
            if "neighbor_list" in te.data:
                te = te.clone()
                te.data["neighbor_list"] = te.data["neighbor_list"] + node_off
            edges = SegmentedLevelStorage.concatenate([mine._edges_group, te])
        system = None
        if mine._system_group is not None and theirs._system_group is not None:
            system = UniformLevelStorage.concatenate([mine._system_group, theirs._system_group])
        object.__setattr__(self, "_storage", MultiLevelStorage(atoms, edges, system, self._storage.schema))

    def append_data(self, data: "AtomicData | Sequence[AtomicData]") -> None:
        items = [data] if isinstance(data, AtomicData) else list(data)
        self.append(Batch.from_data_list(items, device=self.device))

    def _tight(self) -> "Batch":
        a = self._atoms_group
        if a is not None and (a.element_capacity != a.num_elements or a.segment_capacity != a.num_segments):
            return self.index_select(torch.arange(self.num_graphs, device=self.device))
        return self

    def add_key(self, key: str, values: "list[torch.Tensor] | torch.Tensor", level: str = "node",
                overwrite: bool = False) -> None:
        if key in self._storage and not overwrite:
            raise KeyError(f"key {key!r} already exists; pass overwrite=True to replace it")
        self._storage.schema.register(key, level)
        if isinstance(values, (list, tuple)):
            if len(values) != self.num_graphs:
                raise ValueError("add_key expects one value per graph")
            if level == "system":
                values = torch.cat([v if v.dim() >= 1 and v.shape[0] == 1 else v.unsqueeze(0) for v in values], 0)
            else:
                values = torch.cat(list(values), dim=0)
        expected = {"node": self.num_nodes, "edge": self.num_edges, "system": self.num_graphs}[
            {"atoms": "node", "edges": "edge"}.get(level, level) if level in ("atoms", "edges") else level]
        if values.shape[0] != expected:
            raise ValueError(f"{key}: expected {expected} rows at level {level!r}, got {values.shape[0]}")
        self._storage[key] = values.to(self.device)
        if self.keys is not None:
            self.keys.setdefault({"atoms": "node", "edges": "edge"}.get(level, level), set()).add(key)

    # ------------------------------------------------------------------ moves
    def _map(self, fn: Any, device: torch.device | None = None) -> "Batch":
        keys = None if self.keys is None else {k: set(v) for k, v in self.keys.items()}
        return Batch._construct(device=device or self.device, keys=keys,
                                storage=self._storage.map_groups(lambda g: g.apply(fn)),
                                data_class=self._data_class)

    def to(self, device: torch.device | str | None = None, dtype: torch.dtype | None = None,
           non_blocking: bool = False) -> "Batch":
        def fn(t: torch.Tensor) -> torch.Tensor:
            if dtype is not None and t.dtype.is_floating_point:
                t = t.to(dtype)
            return t.to(device, non_blocking=non_blocking) if device is not None else t
        return self._map(fn, torch.device(device) if device is not None else None)

    def clone(self) -> "Batch":
        return self._map(lambda t: t.clone())

    def cpu(self) -> "Batch":
        return self.to("cpu")

    def cuda(self, device: int | None = None, non_blocking: bool = False) -> "Batch":
        return self.to(torch.device("cuda", device) if device is not None else "cuda", non_blocking=non_blocking)

    def contiguous(self) -> "Batch":
        return self._map(lambda t: t.contiguous())

    def pin_memory(self) -> "Batch":
        return self._map(lambda t: t.pin_memory() if t.device.type == "cpu" else t)

    def model_dump(self, **kwargs: Any) -> dict[str, Any]:
        out: dict[str, Any] = {k: v for k, v in self._storage.items()}
        out["batch_idx"] = self.batch_idx
        out["batch_ptr"] = self.batch_ptr
        if kwargs.get("exclude_none"):
            out = {k: v for k, v in out.items() if v is not None}
        return out

    # ------------------------------------------------------- point-to-point IO
    def _wire_fields(self) -> list[tuple[str, str]]:
        out = []
        for gname in ("atoms", "edges", "system"):
            g = self._storage.groups[gname]
            if g is not None:
                out.extend((gname, k) for k in sorted(g.keys()))
        return out

    def isend(self, dst: int, group: Any = None, tag: int = 0, template: "Batch | None" = None) -> "_BatchSendHandle":
        """Non-blocking send.  An empty batch is still sent so the peer's ``irecv`` always completes.

        The receiver posts one message per field of ITS template; with ``template`` given the sender transmits exactly
        that field set (fields this batch lacks go as zeros, fields the template lacks stay behind), so bookkeeping or
        cache fields a stage added to its batch cannot desynchronise the two sides."""
        b = self._tight()
        if template is not None:
            b = b._conformed_to(template)
        header = torch.tensor([b.num_graphs, b.num_nodes, b.num_edges], dtype=torch.int64, device=self.device)
        handles, keep = [], [header]
        handles.append(dist.isend(header, dst, group=group, tag=tag))
        if b.num_graphs > 0:
            seg = torch.cat([b.num_nodes_per_graph, b.num_edges_per_graph]).to(torch.int32).contiguous()
            keep.append(seg)
            handles.append(dist.isend(seg, dst, group=group, tag=tag + 1))
            for i, (gname, k) in enumerate(b._wire_fields()):
                t = b._storage.groups[gname][k]
                if gname == "edges" and b.num_edges == 0:
                    continue
                t = t.to(torch.uint8) if t.dtype == torch.bool else t
                t = t.contiguous()
                keep.append(t)
                handles.append(dist.isend(t, dst, group=group, tag=tag + 2 + i))
        return _BatchSendHandle(handles, keep)

    def _conformed_to(self, template: "Batch") -> "Batch":
        """Shallow copy of this (tight) batch holding exactly the fields of ``template``."""
        rows = {"atoms": self.num_nodes, "edges": self.num_edges, "system": self.num_graphs}
        same = all((self._storage.groups[g] is None) == (template._storage.groups[g] is None) and
                   (self._storage.groups[g] is None or set(self._storage.groups[g].keys()) == set(template._storage.groups[g].keys()))
                   for g in rows)
        if same:
            return self
        out = self.index_select(torch.arange(self.num_graphs, device=self.device))
        for gname, n in rows.items():
            tg, og = template._storage.groups[gname], out._storage.groups[gname]
            if tg is None or og is None:
                continue
            for k in list(og.keys()):
                if k not in tg.data:
                    del og[k]
            for k, ref in tg.data.items():
                if k not in og.data:
                    og[k] = torch.zeros((n,) + tuple(ref.shape[1:]), dtype=ref.dtype, device=self.device)
        return out

    @classmethod
    def irecv(cls, src: int, template: "Batch", device: torch.device | str | None = None, group: Any = None,
              tag: int = 0) -> "_BatchRecvHandle":
        return _BatchRecvHandle(src, template, torch.device(device) if device is not None else template.device,
                                group, tag)

    def send(self, dst: int, group: Any = None, tag: int = 0) -> None:
        self.isend(dst, group=group, tag=tag).wait()

    @classmethod
    def recv(cls, src: int, template: "Batch", device: torch.device | str | None = None, group: Any = None,
             tag: int = 0) -> "Batch":
        return cls.irecv(src, template, device=device, group=group, tag=tag).wait()


class _BatchSendHandle:
    """Keeps the sent tensors alive until ``wait()``."""

    def __init__(self, handles: list, keep: list) -> None:
        self._handles, self._keep = handles, keep

    def wait(self) -> None:
        for h in self._handles:
            if h is not None:
                h.wait()
        self._keep = []


class _BatchRecvHandle:
    """Receives header → segment lengths → fields; buffers are shaped from the template batch."""

    def __init__(self, src: int, template: Batch, device: torch.device, group: Any, tag: int) -> None:
        self.src, self.template, self.device, self.group, self.tag = src, template, device, group, tag
        self.header = torch.zeros(3, dtype=torch.int64, device=device)
        self._h = dist.irecv(self.header, src, group=group, tag=tag)
        self._result: Batch | None = None

    def wait(self) -> Batch:
        if self._result is not None:
            return self._result
        self._h.wait()
        ng, nn, ne = (int(x) for x in self.header.tolist())
        tpl = self.template
        if ng == 0:
            out = tpl.index_select(torch.zeros(0, dtype=torch.long, device=tpl.device)).to(self.device)
            self._result = out
            return out
        seg = torch.zeros(2 * ng, dtype=torch.int32, device=self.device)
        dist.irecv(seg, self.src, group=self.group, tag=self.tag + 1).wait()
        handles, bufs = [], {}
        for i, (gname, k) in enumerate(tpl._wire_fields()):
            ref = tpl._storage.groups[gname].data[k]
            rows = {"atoms": nn, "edges": ne, "system": ng}[gname]
            if gname == "edges" and ne == 0:
                bufs[(gname, k)] = torch.zeros((0,) + tuple(ref.shape[1:]), dtype=ref.dtype, device=self.device)
                continue
            wire_dtype = torch.uint8 if ref.dtype == torch.bool else ref.dtype
            buf = torch.zeros((rows,) + tuple(ref.shape[1:]), dtype=wire_dtype, device=self.device)
            bufs[(gname, k)] = buf
            handles.append(dist.irecv(buf, self.src, group=self.group, tag=self.tag + 2 + i))
        for h in handles:
            h.wait()
        data = {g: {} for g in ("atoms", "edges", "system")}
        for (gname, k), buf in bufs.items():
            ref = tpl._storage.groups[gname].data[k]
            data[gname][k] = buf.to(torch.bool) if ref.dtype == torch.bool else buf
        atoms = SegmentedLevelStorage(data["atoms"], seg[:ng].clone(), num_elements=nn, device=self.device)
        edges = SegmentedLevelStorage(data["edges"], seg[ng:].clone(), num_elements=ne, device=self.device) \
            if tpl._edges_group is not None else None
        system = UniformLevelStorage(data["system"], capacity=ng) if tpl._system_group is not None else None
        keys = None if tpl.keys is None else {k: set(v) for k, v in tpl.keys.items()}
        self._result = Batch._construct(device=self.device, keys=keys,
                                        storage=MultiLevelStorage(atoms, edges, system, tpl._storage.schema.copy()),
                                        data_class=tpl._data_class)
        return self._result
