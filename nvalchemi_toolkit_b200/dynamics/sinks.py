# SPDX-License-Identifier: Apache-2.0
"""Data sinks for graduated / overflowing systems (reference ``nvalchemi/dynamics/sinks.py:43-886``).

``DataSink`` is the interface (``write(batch, mask)``, ``read``, ``drain``, ``zero``, ``capacity``, ``is_full``);
``GPUBuffer`` keeps systems in a pre-allocated device ``Batch`` (masked ``put``), ``HostMemory`` keeps them as CPU
batches, ``ZarrData`` appends them to a Zarr store.
"""
from __future__ import annotations

import abc
from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch


class DataSink(abc.ABC):
    drainable = True

    @abc.abstractmethod
    def write(self, batch: Batch, mask: torch.Tensor | None = None) -> None: ...

    @abc.abstractmethod
    def read(self) -> Batch | None: ...

    @abc.abstractmethod
    def zero(self) -> None: ...

    @abc.abstractmethod
    def __len__(self) -> int: ...

    @property
    @abc.abstractmethod
    def capacity(self) -> int: ...

    @property
    def is_full(self) -> bool:
        return len(self) >= self.capacity

    def drain(self, max_systems: int | None = None) -> Batch | None:
        """Return the stored systems (at most ``max_systems``) and remove them from the sink."""
        data = self.read()
        if data is None or data.num_graphs == 0:
            return None
        if max_systems is None or data.num_graphs <= max_systems:
            self.zero()
            return data
        head = data.index_select(slice(0, max_systems))
        tail = data.index_select(slice(max_systems, data.num_graphs))
        self.zero()
        self.write(tail)
        return head


_TRANSIENT_PREFIXES = ("neighbor_matrix", "num_neighbors")


def _without_transients(batch: Batch) -> Batch:
    """Neighbour matrices are caches of the hooks that built them: their width follows the current neighbour capacity,
    so two batches written at different times need not agree on it.  A sink stores the physical state only."""
    drop = [k for k in batch._storage.keys() if k.startswith(_TRANSIENT_PREFIXES)]
    if not drop:
        return batch
    out = batch.index_select(torch.arange(batch.num_graphs, device=batch.device)) if drop else batch
    for k in drop:
        del out[k]
    return out


def strip_neighbor_caches(batch: Batch) -> Batch:
    """Remove the neighbour-matrix caches from ``batch`` IN PLACE (for a batch that is about to leave its stage: sinks,
    hand-off messages whose field set is fixed by a template)."""
    for k in [k for k in batch._storage.keys() if k.startswith(_TRANSIENT_PREFIXES)]:
        del batch[k]
    return batch


def _masked(batch: Batch, mask: torch.Tensor | None) -> Batch | None:
    if mask is None:
        return _without_transients(batch) if batch.num_graphs else None
    if not bool(mask.any()):
        return None
    return strip_neighbor_caches(batch.index_select(mask))


class GPUBuffer(DataSink):
    """Fixed-capacity device buffer; the storage is allocated lazily from the first batch written."""

    def __init__(self, capacity: int, max_atoms: int, max_edges: int = 0, device: str | torch.device = "cuda") -> None:
        self._capacity, self.max_atoms, self.max_edges = capacity, max_atoms, max_edges
        self.device = torch.device(device)
        self._buf: Batch | None = None

    def write(self, batch: Batch, mask: torch.Tensor | None = None) -> None:
        if self._buf is None:
            self._buf = Batch.empty(num_systems=self._capacity, num_nodes=self.max_atoms * self._capacity,
                                    num_edges=self.max_edges * self._capacity, template=batch, device=self.device)
        src = batch if batch.device == self.device else batch.to(self.device)
        m = torch.ones(src.num_graphs, dtype=torch.bool, device=self.device) if mask is None else mask.to(self.device)
        copied = torch.zeros(src.num_graphs, dtype=torch.bool, device=self.device)
        self._buf.put(src, m, copied_mask=copied)
        if bool((m & ~copied).any()):
            raise RuntimeError("GPUBuffer overflow: not every selected system fits")

    def read(self) -> Batch | None:
        if self._buf is None or self._buf.num_graphs == 0:
            return None
        return self._buf.index_select(torch.arange(self._buf.num_graphs, device=self.device))

    def zero(self) -> None:
        if self._buf is not None:
            self._buf.zero()

    def __len__(self) -> int:
        return 0 if self._buf is None else self._buf.num_graphs

    @property
    def capacity(self) -> int:
        return self._capacity


class HostMemory(DataSink):
    def __init__(self, capacity: int = 1_000_000) -> None:
        self._capacity = capacity
        self._parts: list[Batch] = []
        self._n = 0

    def write(self, batch: Batch, mask: torch.Tensor | None = None) -> None:
        sel = _masked(batch, mask)
        if sel is None:
            return
        if self._n + sel.num_graphs > self._capacity:
            raise RuntimeError("HostMemory sink is full")
        self._parts.append(sel.to("cpu"))
        self._n += sel.num_graphs

    def read(self) -> Batch | None:
        if not self._parts:
            return None
        if len(self._parts) > 1:
            keys = set(self._parts[0]._storage.keys())
            for p in self._parts[1:]:
                keys &= set(p._storage.keys())
            head = self._parts[0].clone()
            for p in self._parts[1:]:
                head.append(p)
            self._parts = [head]
        return self._parts[0]

    def zero(self) -> None:
        self._parts, self._n = [], 0

    def __len__(self) -> int:
        return self._n

    @property
    def capacity(self) -> int:
        return self._capacity


class ZarrData(DataSink):
    """Appends systems to a Zarr v3 store (see :mod:`nvalchemi_toolkit_b200.data.zarr_store`)."""

    drainable = False

    def __init__(self, store: Any, capacity: int = 1_000_000, config: Any = None) -> None:
        from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrReader, AtomicDataZarrWriter

        self.store = store
        self._capacity = capacity
        self._writer = AtomicDataZarrWriter(store, config=config)
        self._reader_cls = AtomicDataZarrReader
        self._n = 0

    def write(self, batch: Batch, mask: torch.Tensor | None = None) -> None:
        sel = _masked(batch, mask)
        if sel is None:
            return
        self._writer.append(sel.to("cpu"))
        self._n += sel.num_graphs

    def read(self) -> Batch | None:
        if self._n == 0:
            return None
        reader = self._reader_cls(self.store)
        dicts = [reader.read(i)[0] for i in range(len(reader))]
        return Batch.from_raw_dicts(dicts, field_levels=reader.field_levels)

    def zero(self) -> None:
        self._writer.reset()
        self._n = 0

    def __len__(self) -> int:
        return self._n

    @property
    def capacity(self) -> int:
        return self._capacity
