# SPDX-License-Identifier: Apache-2.0
"""Counting proxy over ``torch.ops.nvalchemi``: every call of one of this package's native operators is tallied
(benchmarks report the tally as the number of native operator launches in the timed region).  With the bounds-checked
debug mode on (``ops/debug_bounds.py``) every call validates its index arguments on the host first."""
from __future__ import annotations

import torch

_count = 0


class _Ops:
    def __getattr__(self, name: str):
        from nvalchemi_toolkit_b200.ops import _native

        if not _native.available():  # loads the in-tree library on first use
            raise RuntimeError("native extension is not built: run `python -m nvalchemi_toolkit_b200.ops.build`")
        from nvalchemi_toolkit_b200.ops import debug_bounds

        fn = debug_bounds.wrap(name, getattr(torch.ops.nvalchemi, name))  # validates index arguments in debug mode

        def call(*a, **k):
            global _count
            _count += 1
            return fn(*a, **k)

        call.__name__ = name
        object.__setattr__(self, name, call)
        return call


ops = _Ops()


def reset() -> None:
    global _count
    _count = 0


def count() -> int:
    return _count
