# SPDX-License-Identifier: Apache-2.0
"""``SizeAwareSampler``: bin-packing supply of systems for inflight batching.

API and semantics follow the reference (``nvalchemi/dynamics/sampler.py:36-645``): the dataset protocol is
``__len__``, ``__getitem__(i) -> (AtomicData, meta)`` and ``get_metadata(i) -> (num_atoms, num_edges)``; samples are
binned by ``num_atoms // bin_width``; the initial batch is filled round-robin over bins (small and large systems
interleaved); replacements are chosen largest-first within the freed atom / edge / count budget; every handed-out
system is stamped with a unique ``system_id``.  Internally the bookkeeping is a pair of numpy arrays plus a per-bin
cursor instead of deques of indices.
"""
from __future__ import annotations

import random
from typing import Any, Iterator

import numpy as np
import torch

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData
from nvalchemi_toolkit_b200.data.batch import Batch

BYTES_PER_ATOM = 300  # memory heuristic of the reference (dynamics/sampler.py:243-259)


class SizeAwareSampler:
    def __init__(self, dataset: Any, max_atoms: int | None = None, max_edges: int | None = None,
                 max_batch_size: int | None = None, bin_width: int = 1, shuffle: bool = False,
                 max_gpu_memory_fraction: float = 0.8) -> None:
        if max_atoms is None and max_batch_size is None:
            raise ValueError("At least one of max_atoms or max_batch_size must be set.")
        if max_batch_size is not None and max_batch_size < 1:
            raise ValueError(f"max_batch_size must be >= 1, got {max_batch_size}")
        if bin_width < 1:
            raise ValueError(f"bin_width must be >= 1, got {bin_width}")
        if not 0.0 < max_gpu_memory_fraction <= 1.0:
            raise ValueError(f"max_gpu_memory_fraction must be in (0.0, 1.0], got {max_gpu_memory_fraction}")
        for attr, msg in (("__len__", "dataset must implement __len__"), ("__getitem__", "dataset must implement __getitem__"),
                          ("get_metadata", "dataset must implement get_metadata(idx) -> (num_atoms, num_edges)")):
            if not hasattr(dataset, attr):
                raise TypeError(msg)
        self._dataset = dataset
        self._max_atoms, self._max_edges, self._max_batch_size = max_atoms, max_edges, max_batch_size
        self._bin_width, self._shuffle, self._fraction = bin_width, shuffle, max_gpu_memory_fraction
        n = len(dataset)
        meta = np.zeros((n, 2), dtype=np.int64)
        for i in range(n):
            a, e = dataset.get_metadata(i)
            if max_atoms is not None and a > max_atoms:
                raise RuntimeError(f"Sample {i} has {a} atoms, exceeding max_atoms={max_atoms}. This sample can never "
                                   "fit in any batch.")
            if max_edges is not None and e > max_edges:
                raise RuntimeError(f"Sample {i} has {e} edges, exceeding max_edges={max_edges}. This sample can never "
                                   "fit in any batch.")
            meta[i] = (a, e)
        self._meta = meta
        self._consumed = np.zeros(n, dtype=bool)
        self._bins: dict[int, list[int]] = {}
        for i in range(n):
            self._bins.setdefault(int(meta[i, 0]) // bin_width, []).append(i)
        if shuffle:
            for lst in self._bins.values():
                random.shuffle(lst)
        self._next_system_id = 0

    # -- properties -------------------------------------------------------------
    @property
    def max_atoms(self) -> int | None:
        return self._max_atoms

    @property
    def max_edges(self) -> int | None:
        return self._max_edges

    @property
    def max_batch_size(self) -> int | None:
        return self._max_batch_size

    @property
    def exhausted(self) -> bool:
        return bool(self._consumed.all())

    def __len__(self) -> int:
        return int((~self._consumed).sum())

    def __iter__(self) -> Iterator[int]:
        for key in sorted(self._bins):
            for i in self._bins[key]:
                if not self._consumed[i]:
                    yield i

    # -- internals ----------------------------------------------------------------
    def _take(self, idx: int) -> AtomicData:
        data, _ = self._dataset[idx]
        data.add_system_property("system_id", torch.tensor([[self._next_system_id]], dtype=torch.long, device=data.device))
        self._next_system_id += 1
        self._consumed[idx] = True
        return data

    def _gpu_atom_cap(self) -> int | None:
        if not torch.cuda.is_available():
            return None
        total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        usable = int(total * self._fraction) - int(total * 0.2)
        return max(max(usable, 0) // BYTES_PER_ATOM, 1)

    # -- public API -----------------------------------------------------------------
    def build_initial_batch(self) -> Batch:
        cap_atoms = self._max_atoms
        gpu_cap = self._gpu_atom_cap()
        if gpu_cap is not None:
            cap_atoms = gpu_cap if cap_atoms is None else min(cap_atoms, gpu_cap)
        cap_count = self._max_batch_size if self._max_batch_size is not None else float("inf")
        picked: list[AtomicData] = []
        atoms = edges = 0
        active = sorted(self._bins)
        while active and len(picked) < cap_count:
            progressed, still = False, []
            for key in active:
                if len(picked) >= cap_count:
                    break
                remaining = [i for i in self._bins[key] if not self._consumed[i]]
                for i in remaining:
                    a, e = self._meta[i]
                    if cap_atoms is not None and atoms + a > cap_atoms:
                        continue
                    if self._max_edges is not None and edges + e > self._max_edges:
                        continue
                    picked.append(self._take(i))
                    atoms += int(a)
                    edges += int(e)
                    progressed = True
                    break
                if len(remaining) > 1 or (remaining and not self._consumed[remaining[0]]):
                    still.append(key)
            if not progressed:
                break
            active = still
        if not picked:
            raise RuntimeError("Cannot build initial batch: no samples available or constraints too tight.")
        batch = Batch.from_data_list(picked, device=picked[0].device)
        if getattr(batch, "status", None) is None:
            batch.add_key("status", torch.zeros(batch.num_graphs, 1, dtype=torch.long, device=batch.device), "system")
        return batch

    def request_replacement(self, num_atoms: int, num_edges: int) -> AtomicData | None:
        for key in range(num_atoms // self._bin_width, -1, -1):
            for i in self._bins.get(key, ()):
                if not self._consumed[i] and self._meta[i, 0] <= num_atoms and self._meta[i, 1] <= num_edges:
                    return self._take(i)
        return None

    def request_replacements_budget(self, atom_budget: int | None = None, edge_budget: int | None = None,
                                    max_count: int | None = None) -> list[AtomicData]:
        out: list[AtomicData] = []
        for key in sorted(self._bins, reverse=True):
            for i in self._bins[key]:
                if max_count is not None and len(out) >= max_count:
                    return out
                if self._consumed[i]:
                    continue
                a, e = int(self._meta[i, 0]), int(self._meta[i, 1])
                if (atom_budget is not None and a > atom_budget) or (edge_budget is not None and e > edge_budget):
                    continue
                out.append(self._take(i))
                atom_budget = None if atom_budget is None else atom_budget - a
                edge_budget = None if edge_budget is None else edge_budget - e
        return out

    def request_replacements(self, node_counts: torch.Tensor, edge_counts: torch.Tensor) -> list[AtomicData | None]:
        """One replacement per freed slot ``(node_counts[i], edge_counts[i])``; the fit matrix is evaluated on the
        device of the inputs, the choice is first-fit in dataset order."""
        dev = node_counts.device
        meta = torch.as_tensor(self._meta, device=dev)
        avail = torch.as_tensor(~self._consumed, device=dev)
        fits = (meta[:, 0][None] <= node_counts[:, None]) & (meta[:, 1][None] <= edge_counts[:, None])
        out: list[AtomicData | None] = []
        for i in range(node_counts.numel()):
            cand = torch.nonzero(fits[i] & avail)
            if cand.numel() == 0:
                out.append(None)
                continue
            j = int(cand[0, 0])
            avail[j] = False
            out.append(self._take(j))
        return out
