# SPDX-License-Identifier: Apache-2.0
"""Derive a distribution spec from ONE single-process forward of an unmodified model.

Reference: ``nvalchemi/distributed/validate/inference.py`` + ``_core/dispatch_trace.py`` (observe which node-level
gathers and scatters fire in a reference run, translate the firings into a candidate ``MLIPSpec``, keep whatever the
wrapper already declares as a prior).

What the trace measures.  A :class:`DispatchTrace` (a ``TorchFunctionMode``) tags every tensor with the number of
neighbour aggregations its value depends on ("depth").  Inputs have depth 0.  A row gather from a node tensor
(``index_select`` / integer-tensor ``__getitem__`` / ``gather`` along dim 0 of a tensor with one row per atom) keeps
the depth; every other op passes on the maximum depth of its tensor inputs; a row scatter INTO a node-shaped tensor
(``index_add`` / ``scatter_add`` / accumulating ``index_put`` ...) yields depth + 1.  The depth of the energy output is
the number of message passes: an atom's energy then depends on atoms up to ``depth x cutoff`` away, which is the ghost
depth a recomputing halo needs (``MLIPSpec.message_passes``).  The trace also counts the gathers from tensors of depth
>= 1: those are the places where a one-cutoff halo has to refresh ghost rows (``refresh_per_layer``).

From the outputs: tensors with one row per atom are node outputs, the rest are extensive; a per-atom energy among them
means forces can be produced by the framework from weighted node energies (``Consolidation.WEIGHTED_ENERGY``);
forces without per-atom energies mean the model differentiates internally (``Consolidation.DIRECT_MASKED``); if such a
model also sums over atoms itself, those sums must skip ghost rows, which selects ``refresh_per_layer`` (the dispatch
mode masks them and refreshes ghost rows before every gather)."""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field
from typing import Any, Callable

import torch
from torch.overrides import TorchFunctionMode

from nvalchemi_toolkit_b200.distributed.dispatch import _GATHERS, _SCATTERS, _tensors
from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec

_NODE_ENERGY_KEYS = ("atomic_energies", "node_energy", "node_energies", "energies_per_atom")


@dataclass
class TraceSummary:
    n_atoms: int
    message_passes: int = 0
    node_gathers: int = 0            # row gathers from node tensors
    deep_gathers: int = 0            # ... of which from tensors that already depend on a neighbour aggregation
    node_scatters: int = 0           # row scatters that produce node tensors
    system_reductions: int = 0       # scatters of node tensors into fewer rows (per-system sums)
    ops: dict[str, int] = field(default_factory=dict)
    output_depth: dict[str, int] = field(default_factory=dict)
    used_autograd: bool = False

    def describe(self) -> str:
        fired = ", ".join(f"{k} x{v}" for k, v in sorted(self.ops.items()))
        return (f"{self.message_passes} message pass(es); {self.node_gathers} node gathers ({self.deep_gathers} need fresh "
                f"ghost rows), {self.node_scatters} node scatters, {self.system_reductions} per-system reductions; "
                f"autograd inside the model: {'yes' if self.used_autograd else 'no'}; ops: {fired or 'none'}")


class DispatchTrace(TorchFunctionMode):
    def __init__(self, n_atoms: int) -> None:
        super().__init__()
        self.summary = TraceSummary(int(n_atoms))
        self._depth: dict[int, tuple[Any, int]] = {}

    # ---- depth bookkeeping
    def depth(self, t: Any) -> int:
        hit = self._depth.get(id(t)) if isinstance(t, torch.Tensor) else None
        return hit[1] if hit is not None and hit[0]() is t else 0

    def _tag(self, t: torch.Tensor, d: int) -> None:
        if d > 0:
            key = id(t)
            self._depth[key] = (weakref.ref(t, lambda _r, k=key, m=self._depth: m.pop(k, None)), d)

    def _is_node(self, t: Any) -> bool:
        return isinstance(t, torch.Tensor) and t.dim() >= 1 and t.shape[0] == self.summary.n_atoms

    @staticmethod
    def _row_op(name: str, args: tuple, kwargs: dict) -> bool:
        x = args[0]
        if name == "__getitem__":
            idx = args[1]
            first = idx[0] if isinstance(idx, tuple) and idx else idx
            return isinstance(first, torch.Tensor) and first.dtype in (torch.int64, torch.int32)
        if name.startswith("index_put"):
            accumulate = args[3] if len(args) > 3 else kwargs.get("accumulate", False)
            return bool(accumulate)
        dim = args[1] if len(args) > 1 else kwargs.get("dim")
        return isinstance(dim, int) and isinstance(x, torch.Tensor) and (dim == 0 or dim == -x.dim())

    def __torch_function__(self, func: Callable, types: Any, args: tuple = (), kwargs: dict | None = None) -> Any:
        kwargs = kwargs or {}
        name = getattr(func, "__name__", "")
        s = self.summary
        if name in ("grad", "backward") and getattr(func, "__module__", "").startswith("torch.autograd"):
            s.used_autograd = True
        d_in = max([self.depth(t) for t in _tensors(args)] + [self.depth(t) for t in _tensors(kwargs)] + [0])
        out = func(*args, **kwargs)
        d_out = d_in
        if args and isinstance(args[0], torch.Tensor) and name in _GATHERS and self._is_node(args[0]) and self._row_op(name, args, kwargs):
            s.node_gathers += 1
            s.deep_gathers += int(self.depth(args[0]) >= 1)
            s.ops[name] = s.ops.get(name, 0) + 1
        elif args and isinstance(args[0], torch.Tensor) and name in _SCATTERS and self._row_op(name, args, kwargs):
            src = next((t for t in list(_tensors(args[1:])) + list(_tensors(kwargs)) if t.is_floating_point()), None)
            result = out if isinstance(out, torch.Tensor) else args[0]
            if self._is_node(result):
                # (a source with one row per atom can only mean a graph with as many edges as atoms: still an aggregation)
                s.node_scatters += 1
                d_out = d_in + 1
                s.ops[name] = s.ops.get(name, 0) + 1
            elif self._is_node(src):
                s.system_reductions += 1
                s.ops[name] = s.ops.get(name, 0) + 1
        for t in _tensors(out):
            self._tag(t, d_out)
        if name.endswith("_") and args and isinstance(args[0], torch.Tensor):
            self._tag(args[0], max(d_out, self.depth(args[0])))
        return out


def trace_model(model: Callable[[Any], dict], batch: Any) -> tuple[dict, TraceSummary]:
    """Run ``model(batch)`` under a :class:`DispatchTrace`.  Returns the outputs and the summary."""
    n = int(batch.positions.shape[0])
    if hasattr(model, "make_neighbor_hooks") and getattr(batch, "neighbor_matrix", None) is None and \
            getattr(batch, "edge_index", None) is None:
        from types import SimpleNamespace

        for hook in model.make_neighbor_hooks():  # the list is an input of the model, built outside the trace
            hook(SimpleNamespace(batch=batch), None)
    with DispatchTrace(n) as tr:
        out = model(batch)
    s = tr.summary
    for k, v in (out.items() if isinstance(out, dict) else []):
        if isinstance(v, torch.Tensor):
            s.output_depth[k] = tr.depth(v)
    energy_like = [s.output_depth[k] for k in s.output_depth if k in ("energy", "energies") + _NODE_ENERGY_KEYS]
    s.message_passes = max(energy_like or list(s.output_depth.values()) or [0])
    return out, s


def infer_spec(model: Any, batch: Any, name: str | None = None, prior: MLIPSpec | None = None) -> tuple[MLIPSpec, TraceSummary]:
    """Candidate spec for ``model`` from one forward on ``batch`` (single process, any device).

    ``prior``: a declared spec; its fields win wherever they differ from the dataclass defaults, the trace fills in the
    rest (reference ``inference.py``: "missing fields are inferred; provided fields are kept verbatim")."""
    out, s = trace_model(model, batch)
    n = s.n_atoms
    tensors = {k: v for k, v in out.items() if isinstance(v, torch.Tensor)}
    node_outputs = tuple(k for k, v in tensors.items() if v.dim() >= 1 and v.shape[0] == n and n != int(getattr(batch, "num_graphs", -1)))
    extensive = tuple(k for k in tensors if k not in node_outputs)
    node_energy_key = next((k for k in _NODE_ENERGY_KEYS if k in node_outputs), None)
    if node_energy_key is not None:
        consolidation = Consolidation.WEIGHTED_ENERGY
    else:
        consolidation = Consolidation.DIRECT_MASKED
    passes = s.message_passes
    notes = f"inferred from a trace: {s.describe()}"
    if passes == 0 and getattr(getattr(model, "model_config", None), "neighbor_config", None) is not None:
        passes = 1  # the neighbour list is consumed inside an operator the trace cannot see into: one hop at least
        notes += "; no gather / scatter was visible (opaque operator): one message pass assumed"
    # Without per-atom energies the framework cannot weight the energy by ownership afterwards: the per-system sums
    # INSIDE the model must skip ghost rows, which only the dispatch mode does (it also refreshes ghost rows before each
    # gather, so one cutoff of ghosts suffices).  It needs the gathers and scatters to be visible to it.
    refresh = node_energy_key is None and s.node_scatters > 0 and s.system_reductions > 0
    if refresh:
        # the masked sums make the model's own energy the owned-atom energy; its position gradient still lands partly on
        # ghost rows and is returned to the owners by the reverse halo of the weighted-energy consolidation
        consolidation = Consolidation.WEIGHTED_ENERGY
        notes += "; no per-atom energy output: per-layer refresh with owned-only reductions selected"
    spec = MLIPSpec(name=name or f"inferred:{type(model).__name__}", message_passes=passes, consolidation=consolidation,
                    refresh_per_layer=refresh,
                    node_energy_key=node_energy_key or "atomic_energies", node_outputs=node_outputs or ("forces",),
                    extensive_outputs=extensive or ("energy",), notes=notes)
    if prior is not None:
        blank = MLIPSpec(name=prior.name)
        keep = {f: getattr(prior, f) for f in ("message_passes", "consolidation", "node_energy_key", "requires_full_list",
                                               "node_outputs", "extensive_outputs", "needs_total_charge", "refresh_per_layer",
                                               "storage_policy", "extra") if getattr(prior, f) != getattr(blank, f)}
        spec = spec.with_(name=prior.name, compile=prior.compile, **keep)
    return spec, s
