# SPDX-License-Identifier: Apache-2.0
"""Adapter for UMA / eSCN backbones (optional dependency ``fairchem-core``).

Reference: ``nvalchemi/models/uma.py:145-1556``: tensor-native input (no ``ase`` round trip): positions, atomic
numbers, cell, per-system ``charge`` / ``spin`` / task name, and a COO edge list with cell offsets; outputs energy,
forces, stress.  The adapter accepts any ``nn.Module`` that maps such a dictionary to ``{"energy", "forces"?, "stress"?}``;
forces and stresses it does not return itself are derived by autograd.  ``from_checkpoint`` needs ``fairchem-core``.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200._optional import OptionalDependency
from nvalchemi_toolkit_b200.models._utils import prepare_strain
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat


class UMAWrapper(nn.Module, BaseModelMixin):
    def __init__(self, model: nn.Module, cutoff: float = 6.0, task_name: str = "omat", direct_forces: bool = False) -> None:
        super().__init__()
        self.model, self.cutoff, self.task_name, self.direct_forces = model, float(cutoff), task_name, direct_forces
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress"}),
            autograd_outputs=frozenset() if direct_forces else frozenset({"forces", "stress"}),
            autograd_inputs=frozenset() if direct_forces else frozenset({"positions"}),
            optional_inputs=frozenset({"cell", "pbc", "charge", "spin", "neighbor_list_shifts"}), supports_pbc=True,
            neighbor_config=NeighborConfig(cutoff=self.cutoff, format=NeighborListFormat.COO, half_list=False),
            active_outputs={"energy", "forces"})

    @classmethod
    def from_checkpoint(cls, name_or_path: str, device: str | torch.device = "cpu", **kw: Any) -> "UMAWrapper":
        fairchem = OptionalDependency.UMA.import_module()
        unit = fairchem.pretrained_mlip.get_predict_unit(name_or_path, device=str(device))
        return cls(unit.model, **kw)

    def adapt_input(self, data: Any, **kwargs: Any) -> dict[str, Any]:
        pos = data.positions
        n = pos.shape[0]
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        batch = data.batch_idx.long() if hasattr(data, "batch_idx") else torch.zeros(n, dtype=torch.long, device=pos.device)
        nl = data.neighbor_list
        keep = (nl < n).all(dim=1)
        nl = nl[keep]
        cell = getattr(data, "cell", None)
        unit = getattr(data, "neighbor_list_shifts", None)
        out = {"pos": pos, "atomic_numbers": data.atomic_numbers.long(), "batch": batch, "natoms": data.num_nodes_per_graph.long()
               if hasattr(data, "num_nodes_per_graph") else torch.tensor([n], device=pos.device),
               "edge_index": nl.t().contiguous().flip(0),  # (source = neighbour, target = centre)
               "cell": cell.reshape(nb, 3, 3) if cell is not None else None,
               "cell_offsets": unit[keep].to(pos.dtype) if unit is not None else pos.new_zeros(nl.shape[0], 3),
               "nedges": torch.bincount(batch[nl[:, 0]], minlength=nb),
               "charge": getattr(data, "charge", None), "spin": getattr(data, "spin", None),
               "dataset": [self.task_name] * nb}
        for key in ("charge", "spin"):
            if out[key] is None:
                out[key] = torch.zeros(nb, dtype=torch.long, device=pos.device)
        return out

    def forward(self, data: Any, **kwargs: Any) -> dict:
        active = set(self.model_config.active_outputs)
        want_f = "forces" in active and not self.direct_forces
        want_s = "stress" in active and not self.direct_forces
        pos0, cell0 = data.positions, getattr(data, "cell", None)
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        with torch.enable_grad() if (want_f or want_s or pos0.requires_grad) else torch.no_grad():
            leaf = pos0 if pos0.requires_grad else pos0.detach().requires_grad_(want_f or want_s)
            strain = None
            if want_s and cell0 is not None:
                spos, scell, strain = prepare_strain(leaf, cell0.detach().reshape(nb, 3, 3), data.batch_idx)
                data["positions"], data["cell"] = spos, scell.reshape(cell0.shape)
            elif leaf is not pos0:
                data["positions"] = leaf
            try:
                res = self.model(self.adapt_input(data))
            finally:
                data["positions"] = pos0
                if strain is not None:
                    data["cell"] = cell0
            energy = res["energy"].reshape(nb)
            out: dict[str, Any] = {"energy": energy, "forces": res.get("forces"), "stress": res.get("stress")}
            if want_f or want_s:
                wrt = [leaf] + ([strain] if strain is not None else [])
                grads = torch.autograd.grad(energy.sum(), wrt, create_graph=self.training, retain_graph=self.training)
                if want_f:
                    out["forces"] = -grads[0]
                if strain is not None:
                    vol = torch.linalg.det(cell0.detach().reshape(nb, 3, 3)).abs().clamp_min(1e-30)
                    out["stress"] = grads[1] / vol[:, None, None]
        return self.adapt_output(out, data)

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed.spec import MLIPSpec, StrategyKind

        kind = StrategyKind.GRAPH_PARTITION if strategy is not None and str(getattr(strategy, "value", strategy)) == \
            "graph_partition" else StrategyKind.HALO
        layers = int(getattr(self.model, "num_layers", 4))
        return MLIPSpec("uma", strategy=kind, message_passes=layers)
