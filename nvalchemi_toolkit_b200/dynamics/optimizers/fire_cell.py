# SPDX-License-Identifier: Apache-2.0
"""``FIREVariableCell``: FIRE on positions plus a unit-cell filter driven by the stress
(reference ``nvalchemi/dynamics/optimizers/fire.py`` ``FIREVariableCell``; cell alignment via ``AlignCellHook``)."""
from __future__ import annotations

from typing import Any

import torch

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics.optimizers.fire import FIRE
from nvalchemi_toolkit_b200.dynamics.optimizers.fire2 import _CellFilterMixin


class FIREVariableCell(FIRE, _CellFilterMixin):
    __needs_keys__ = {"forces", "stress"}
    __provides_keys__ = {"positions", "velocities", "cell"}

    def __init__(self, model: Any, dt: float, *a: Any, cell_factor: float | None = None, **k: Any) -> None:
        super().__init__(model, dt, *a, **k)
        self.cell_factor = cell_factor
        model.model_config.active_outputs = set(model.model_config.active_outputs) | {"stress"}

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor]:
        st = super()._make_new_state(n, template_batch)
        dev, dtype = template_batch.device, template_batch.positions.dtype
        st["cell_velocity"] = torch.zeros(n, 3, 3, dtype=dtype, device=dev)
        for k in ("alpha", "dt", "n_steps_positive", "vf", "vv", "ff"):
            st["cell_" + k] = st[k].clone()
        return st

    def pre_update(self, batch: Batch) -> None:
        s = self._state
        m = batch.num_graphs

        def step_cell(cell_force: torch.Tensor) -> None:
            idx = torch.arange(m, device=batch.device, dtype=torch.int32).repeat_interleave(3)
            ones = torch.ones(3 * m, dtype=cell_force.dtype, device=batch.device)
            _ops.fire_step(batch.cell.reshape(3 * m, 3), s["cell_velocity"].reshape(3 * m, 3),
                           cell_force.reshape(3 * m, 3).contiguous(), ones, s["cell_alpha"], s["cell_dt"],
                           s["cell_n_steps_positive"], s["alpha_start"], s["f_alpha"], s["dt_min"], s["dt_max"],
                           s["maxstep"], s["n_min"], s["f_dec"], s["f_inc"], s["uphill_flag"], vf=s["cell_vf"],
                           vv=s["cell_vv"], ff=s["cell_ff"], batch_idx=idx)

        self._cell_step(batch, step_cell)
        super().pre_update(batch)
