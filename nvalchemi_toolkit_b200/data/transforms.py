# SPDX-License-Identifier: Apache-2.0
"""Composition of data transforms.

Two kinds exist (reference ``nvalchemi/data/transforms/compose.py:43-260``): a *sample* transform maps
``(AtomicData, metadata) -> (AtomicData, metadata)`` and runs inside a ``Dataset``; a *batch* transform maps
``Batch -> Batch`` and runs on collated batches.  :class:`Compose` chains transforms of ONE kind.  The kind is read from
the annotation of each callable's first positional parameter (``AtomicData`` or ``Batch``); callables without an
annotation fit either kind; any other annotation, or a mixture of the two kinds, is rejected when the chain is built,
not when the first sample arrives."""
from __future__ import annotations

import inspect
from typing import Any, Callable, Sequence, get_type_hints

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData
from nvalchemi_toolkit_b200.data.batch import Batch


def transform_kind(transforms: Sequence[Callable]) -> str | None:
    """``"sample"``, ``"batch"`` or ``None`` (nothing annotated).  Raises ``TypeError`` for a non-callable entry, a first
    parameter annotated with something else, or typed entries that disagree."""
    kind: str | None = None
    decided_by = -1
    for i, fn in enumerate(transforms):
        if not callable(fn):
            raise TypeError(f"Compose: entry {i} is not callable ({type(fn).__name__})")
        target = fn if (inspect.isfunction(fn) or inspect.ismethod(fn) or inspect.isbuiltin(fn)) else getattr(type(fn), "__call__", fn)
        try:
            hints = get_type_hints(target)
            params = [p for p in inspect.signature(fn).parameters.values()
                      if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        except Exception:  # noqa: BLE001 - builtins, C callables, unresolvable forward references: treated as untyped
            continue
        if not params or params[0].name not in hints:
            continue
        first = hints[params[0].name]
        if first is AtomicData:
            this = "sample"
        elif first is Batch:
            this = "batch"
        else:
            raise TypeError(f"Compose: entry {i} ({fn!r}) takes {first!r} first; a sample transform takes AtomicData, a "
                            "batch transform takes Batch")
        if kind is None:
            kind, decided_by = this, i
        elif kind != this:
            raise TypeError(f"Compose: entry {decided_by} is a {kind} transform, entry {i} a {this} transform; "
                            "they cannot share one chain")
    return kind


class Compose:
    """Chain of transforms of one kind.  Called with ``(data, metadata)`` it runs sample transforms and returns the pair;
    called with one argument it runs batch transforms and returns the batch."""

    def __init__(self, transforms: Sequence[Callable]) -> None:
        self.transforms = list(transforms)
        self.kind = transform_kind(self.transforms)

    def __call__(self, data: Any, meta: dict[str, Any] | None = None) -> Any:
        if meta is None:
            if self.kind == "sample":
                raise TypeError("this chain holds sample transforms: call it with (data, metadata)")
            for t in self.transforms:
                data = t(data)
            return data
        if self.kind == "batch":
            raise TypeError("this chain holds batch transforms: call it with the batch only")
        for t in self.transforms:
            data, meta = t(data, meta)
        return data, meta

    def __add__(self, other: "Compose | Callable") -> "Compose":
        return Compose(self.transforms + (other.transforms if isinstance(other, Compose) else [other]))

    def __len__(self) -> int:
        return len(self.transforms)

    def __iter__(self):
        return iter(self.transforms)

    def __repr__(self) -> str:
        names = ", ".join(getattr(t, "__name__", type(t).__name__) for t in self.transforms)
        return f"Compose[{self.kind or 'untyped'}]({names})"
