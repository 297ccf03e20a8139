# SPDX-License-Identifier: Apache-2.0
"""Per-output declarations for the consolidation of a decomposed evaluation.

Reference: ``nvalchemi/distributed/output_kinds.py`` (``OutputKind``, ``Reduce``, ``OutputSpec``).  A model output has a
shape (one row per atom, one row per system, or neither) and a combination rule (each rank holds a partial sum, or
every rank already holds the final value).  ``MLIPSpec`` stores the result as two name lists (``node_outputs``,
``extensive_outputs``); :func:`lower_outputs` turns the per-output declarations into those lists, so consolidation and
the serialised form of a spec do not change."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Mapping


class OutputKind(Enum):
    PER_NODE = "per_node"    # one row per atom (owned + ghost rows on the padded sub-domain)
    PER_GRAPH = "per_graph"  # one row per system
    GLOBAL = "global"        # already the same on every rank: passed through
    UNKNOWN = "unknown"      # undeclared: consolidation falls back to the row count


class Reduce(Enum):
    NONE = "none"              # the default of the kind (owned rows of a node output; a system output passes through)
    ALL_REDUCE = "all_reduce"  # every rank holds a partial sum
    OWNED_ONLY = "owned_only"  # already final on every rank: owned rows / pass-through, no collective


@dataclass(frozen=True)
class OutputSpec:
    kind: OutputKind = OutputKind.UNKNOWN
    reduce: Reduce = Reduce.NONE


def lower_outputs(outputs: Mapping[str, OutputSpec]) -> tuple[tuple[str, ...], tuple[str, ...]]:
    """``(node_outputs, extensive_outputs)`` for ``MLIPSpec``.  A node output that asks for an all-reduce is refused: rows
    of different ranks are different atoms, there is nothing to add."""
    node, extensive = [], []
    for name, spec in outputs.items():
        if not isinstance(spec, OutputSpec):
            raise TypeError(f"outputs[{name!r}] must be an OutputSpec, got {type(spec).__name__}")
        if spec.kind == OutputKind.PER_NODE:
            if spec.reduce == Reduce.ALL_REDUCE:
                raise ValueError(f"output {name!r}: a per-node output cannot be all-reduced (rows of different ranks are "
                                 "different atoms); ghost-row contributions return to their owners by the reverse halo")
            node.append(name)
        elif spec.reduce == Reduce.ALL_REDUCE:
            if spec.kind == OutputKind.GLOBAL:
                raise ValueError(f"output {name!r}: GLOBAL means already final on every rank; it cannot also be all-reduced")
            extensive.append(name)
    return tuple(node), tuple(extensive)
