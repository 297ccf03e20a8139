# SPDX-License-Identifier: Apache-2.0
"""Fixed-shape padding of the per-rank graph, so that a captured CUDA graph (or any shape-specialised executor) can be
replayed across MD steps although the number of owned + ghost atoms and of edges changes every step.

Reference: ``nvalchemi/distributed/graph_padder.py:60-593`` (``resolve_cap``, ``cap_agreement_group``, ``GraphPadder``
protocol, ``COOPadder``, ``DensePadder``, ``DenseBatchPadder``).  The reference pads for ``torch.compile``; here the
consumer is stream capture: tensor addresses and shapes must not change between replays, so capacities only grow, grow
in buckets, and grow on every rank at once (a rank that re-captures alone would issue a different sequence of
collectives than its peers).

Dead atoms carry ``Z = 0`` and zero position, join the last system, have no neighbours and are referenced by no real
edge; dead edges are self-loops on the last dead atom with lattice shift ``(1, 0, 0)`` (a zero edge vector would produce
NaNs in spherical harmonics).  Their outputs are dropped by :meth:`unpad` / by the owned-row consolidation.
"""
from __future__ import annotations

import contextvars
from contextlib import contextmanager
from typing import Any, Iterator, Protocol, runtime_checkable

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.level_storage import MultiLevelStorage, SegmentedLevelStorage, UniformLevelStorage

__all__ = ["GraphPadder", "COOPadder", "DensePadder", "DenseBatchPadder", "resolve_cap", "cap_agreement_group"]

_CAP_AGREEMENT: contextvars.ContextVar[tuple[Any, Any] | None] = contextvars.ContextVar("nva_cap_agreement", default=None)


@contextmanager
def cap_agreement_group(group: Any, device: Any) -> Iterator[None]:
    """Inside this scope :func:`resolve_cap` sizes every capacity from the MAXIMUM need over the ranks of ``group``."""
    token = _CAP_AGREEMENT.set((group, device))
    try:
        yield
    finally:
        _CAP_AGREEMENT.reset(token)


def resolve_cap(state: dict[str, int], key: str, real: int, *, initial_factor: float = 1.15, grow_factor: float = 1.30,
                stride: int = 16, extra: int = 0, strict_gt: bool = True) -> int:
    """Grow-only capacity for ``key``: at least ``real + extra`` (strictly more when ``strict_gt`` is false, for
    layouts that keep a dead row in the last slot), sized with ``initial_factor`` head-room on first sight and with
    ``grow_factor`` on overflow, always a multiple of ``stride``.  ``state`` persists between calls."""
    need = int(real) + int(extra)
    agree = _CAP_AGREEMENT.get()
    if agree is not None:
        import torch.distributed as dist

        group, device = agree
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            t = torch.tensor([need], device=device, dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            need = int(t.item())

    def bucket(x: int, factor: float) -> int:
        return -(-(int(x * factor) + 1) // stride) * stride

    cap = state.get(key)
    if cap is None:
        cap = bucket(need, initial_factor)
    elif (need > cap) if strict_gt else (need >= cap):
        cap = max(stride, bucket(need, grow_factor))
    state[key] = cap
    return cap


@runtime_checkable
class GraphPadder(Protocol):
    def pad(self, data: Any, cap_state: dict[str, int], cap_atoms: bool = True) -> Any: ...

    def unpad(self, output: Any, n_real: int | None = None) -> Any: ...


def _groups(batch: Batch) -> tuple[dict, dict, dict]:
    a, e, s = batch._atoms_group, batch._edges_group, batch._system_group
    return ({k: a[k] for k in a.keys()} if a is not None else {}, {k: e[k] for k in e.keys()} if e is not None else {},
            {k: s[k] for k in s.keys()} if s is not None else {})


def _pad_rows(t: torch.Tensor, n: int, fill: Any = 0) -> torch.Tensor:
    if t.shape[0] >= n:
        return t
    tail = t.new_full((n - t.shape[0],) + tuple(t.shape[1:]), fill)
    return torch.cat([t, tail])


def _rebuild(batch: Batch, node: dict, edge: dict, system: dict, n_extra_nodes: int, n_extra_edges: int) -> Batch:
    """Batch with the given concatenated fields; the extra rows join the last graph."""
    dev = batch.device
    nn_ = batch.num_nodes_per_graph.to(torch.int32).clone()
    nn_[-1] += n_extra_nodes
    atoms = SegmentedLevelStorage(node, nn_.to(dev), num_elements=int(nn_.sum()), device=dev)
    edges = None
    if edge:
        ne = (batch.edge_ptr[1:] - batch.edge_ptr[:-1]).to(torch.int32).clone()
        ne[-1] += n_extra_edges
        edges = SegmentedLevelStorage(edge, ne.to(dev), num_elements=int(ne.sum()), device=dev)
    sysg = UniformLevelStorage(system, capacity=batch.num_graphs)
    storage = MultiLevelStorage(atoms, edges, sysg, batch._storage.schema)
    keys = {"node": set(node), "edge": set(edge), "system": set(system)}
    out = Batch._construct(device=dev, keys=keys, storage=storage, data_class=batch._data_class)
    if hasattr(batch, "_dd"):
        object.__setattr__(out, "_dd", batch._dd)
    return out


def _strip(output: Any, n_real: int | None, n_cap: int | None, keys: tuple[str, ...] | None = None) -> Any:
    if n_real is None or not isinstance(output, dict):
        return output
    res = {}
    for k, v in output.items():
        node_level = isinstance(v, torch.Tensor) and v.dim() >= 1 and (v.shape[0] == n_cap if n_cap is not None else False)
        res[k] = v[:n_real] if node_level and (keys is None or k in keys) else v
    return res


class COOPadder:
    """Pads a batch whose graph is a COO ``neighbor_list [E, 2]`` (+ ``neighbor_list_shifts``) to fixed atom and edge
    capacities.  Edges that already point at or beyond the real atom count (a model's own sentinel rows) are re-routed
    to the dead atom as well."""

    def __init__(self, atom_factor: float = 1.15, edge_factor: float = 1.35, grow_factor: float = 1.30, stride: int = 16,
                 list_key: str = "neighbor_list", shifts_key: str = "neighbor_list_shifts") -> None:
        self.atom_factor, self.edge_factor, self.grow_factor, self.stride = atom_factor, edge_factor, grow_factor, stride
        self.list_key, self.shifts_key = list_key, shifts_key
        self._n_cap: int | None = None

    def pad(self, data: Batch, cap_state: dict[str, int], cap_atoms: bool = True) -> Batch:
        node, edge, system = _groups(data)
        n_real, e_real = data.num_nodes, data.num_edges
        n_cap = resolve_cap(cap_state, "atoms", n_real, initial_factor=self.atom_factor, grow_factor=self.grow_factor,
                            stride=self.stride, strict_gt=False) if cap_atoms else n_real + 1
        e_cap = resolve_cap(cap_state, "edges", e_real, initial_factor=self.edge_factor, grow_factor=self.grow_factor,
                            stride=self.stride)
        self._n_cap = n_cap
        dead = n_cap - 1
        node = {k: _pad_rows(v, n_cap) for k, v in node.items()}
        out_edge = {}
        for k, v in edge.items():
            if k == self.list_key:
                nl = _pad_rows(v, e_cap, dead).clone()
                nl[(nl >= n_real).any(dim=1)] = dead
                out_edge[k] = nl
            elif k == self.shifts_key:
                sh = _pad_rows(v, e_cap, 0).clone()
                sh[e_real:, 0] = 1
                out_edge[k] = sh
            else:
                out_edge[k] = _pad_rows(v, e_cap)
        return _rebuild(data, node, out_edge, system, n_cap - n_real, e_cap - e_real)

    def unpad(self, output: Any, n_real: int | None = None) -> Any:
        return _strip(output, n_real, self._n_cap)


class DensePadder:
    """Pads per-atom tensors of a dense ``(N, K)`` neighbour-matrix graph held in a plain dict: every field in
    ``row_pads`` grows to the atom capacity with its fill value (``DensePadder.LAST_SYSTEM`` repeats the last system's
    label), and matrix entries ``>= n_real`` (the model's sentinel for unused slots) are re-pointed to the dead row."""

    LAST_SYSTEM = object()

    def __init__(self, count_key: str = "positions", nbmat_key: str = "neighbor_matrix", row_pads: dict[str, Any] | None = None,
                 atom_output_keys: tuple[str, ...] = ("forces", "atomic_energies", "charges"), initial_factor: float = 1.15,
                 grow_factor: float = 1.30, stride: int = 16) -> None:
        self.count_key, self.nbmat_key = count_key, nbmat_key
        self.row_pads = dict(row_pads) if row_pads is not None else {}
        self.atom_output_keys = tuple(atom_output_keys)
        self.initial_factor, self.grow_factor, self.stride = initial_factor, grow_factor, stride
        self._n_cap: int | None = None

    def pad(self, data: dict, cap_state: dict[str, int], cap_atoms: bool = True) -> dict:
        n_real = int(data[self.count_key].shape[0])
        n_cap = resolve_cap(cap_state, "atoms", n_real, initial_factor=self.initial_factor, grow_factor=self.grow_factor,
                            stride=self.stride, strict_gt=False) if cap_atoms else n_real + 1
        self._n_cap = n_cap
        out = dict(data)
        for k, v in data.items():
            if not isinstance(v, torch.Tensor) or v.dim() < 1 or v.shape[0] != n_real:
                continue
            if k == self.nbmat_key:
                m = _pad_rows(v, n_cap, n_cap - 1).clone()
                m[m >= n_real] = n_cap - 1
                out[k] = m
            else:
                fill = self.row_pads.get(k, 0)
                if fill is DensePadder.LAST_SYSTEM:
                    fill = v[-1].item() if n_real else 0
                out[k] = _pad_rows(v, n_cap, fill)
        return out

    def unpad(self, output: Any, n_real: int | None = None) -> Any:
        return _strip(output, n_real, self._n_cap, self.atom_output_keys)


class DenseBatchPadder:
    """Pads a :class:`Batch` whose graph is the MATRIX neighbour format (``neighbor_matrix [N, K]``, ``num_neighbors``,
    ``neighbor_matrix_shifts``) to a fixed atom capacity; optionally also to a fixed neighbour capacity ``K``.  Dead
    rows have ``num_neighbors = 0`` and unused slots point at the dead row."""

    def __init__(self, nbmat_key: str = "neighbor_matrix", count_key: str = "num_neighbors",
                 shifts_key: str = "neighbor_matrix_shifts", initial_factor: float = 1.15, grow_factor: float = 1.30,
                 stride: int = 16, pad_neighbors: bool = False) -> None:
        self.nbmat_key, self.count_key, self.shifts_key = nbmat_key, count_key, shifts_key
        self.initial_factor, self.grow_factor, self.stride, self.pad_neighbors = initial_factor, grow_factor, stride, pad_neighbors
        self._n_cap: int | None = None

    def pad(self, data: Batch, cap_state: dict[str, int], cap_atoms: bool = True) -> Batch:
        node, edge, system = _groups(data)
        n_real = data.num_nodes
        n_cap = resolve_cap(cap_state, "atoms", n_real, initial_factor=self.initial_factor, grow_factor=self.grow_factor,
                            stride=self.stride, strict_gt=False) if cap_atoms else n_real + 1
        self._n_cap = n_cap
        dead = n_cap - 1
        k_cap = None
        if self.pad_neighbors and self.nbmat_key in node:
            k_cap = resolve_cap(cap_state, "neighbors", node[self.nbmat_key].shape[1], initial_factor=1.0,
                                grow_factor=self.grow_factor, stride=8)

        def widen(v: torch.Tensor, fill: Any) -> torch.Tensor:
            if k_cap is None or v.shape[1] >= k_cap:
                return v
            return torch.cat([v, v.new_full((v.shape[0], k_cap - v.shape[1]) + tuple(v.shape[2:]), fill)], dim=1)

        out = {}
        for k, v in node.items():
            if k == self.nbmat_key:
                m = _pad_rows(widen(v, dead), n_cap, dead).clone()
                cnt = node.get(self.count_key)
                if cnt is not None:  # unused slots of real rows
                    slot = torch.arange(m.shape[1], device=m.device)[None, :]
                    m[slot >= _pad_rows(cnt, n_cap, 0).long()[:, None]] = dead
                m[m >= n_real] = dead
                out[k] = m
            elif k == self.shifts_key:
                out[k] = _pad_rows(widen(v, 0), n_cap)
            else:
                out[k] = _pad_rows(v, n_cap)
        return _rebuild(data, out, edge, system, n_cap - n_real, 0)

    def unpad(self, output: Any, n_real: int | None = None) -> Any:
        return _strip(output, n_real, self._n_cap)
