# SPDX-License-Identifier: Apache-2.0
"""``WrapPeriodicHook``: wraps positions back into the cell (reference ``nvalchemi/hooks/periodic.py:42-218``)."""
from __future__ import annotations

from enum import Enum
from typing import Any

from nvalchemi_toolkit_b200.dynamics import _ops


def wrap_positions(positions, cell, batch_idx, pbc=None):
    return _ops.wrap_positions(positions, cell, batch_idx, pbc)


class WrapPeriodicHook:
    def __init__(self, frequency: int = 1, stage: Enum | None = None) -> None:
        self.frequency, self.stage = frequency, stage

    def on_register(self, owner: Any) -> None:
        if self.stage is None:
            from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage

            self.stage = DynamicsStage.AFTER_POST_UPDATE

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        cell, pbc = getattr(b, "cell", None), getattr(b, "pbc", None)
        if cell is None or pbc is None:
            return
        seen = getattr(self, "_pbc_seen", None)
        if seen is None or seen[0] is not pbc or seen[1] != pbc._version:  # one host read per pbc tensor, not per step
            self._pbc_seen = seen = (pbc, pbc._version, bool(pbc.any()))
        if not seen[2]:
            return
        b.positions.copy_(_ops.wrap_positions(b.positions, cell.reshape(-1, 3, 3), b.batch_idx, pbc.reshape(-1, 3)))
