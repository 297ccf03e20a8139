# SPDX-License-Identifier: Apache-2.0
"""``MACEWrapper``: the ``BaseModelMixin`` adapter for a MACE network.

Contract as in the reference (``nvalchemi/models/mace.py:518-1158``): outputs ``energy, forces, stress, hessian,
atomic_energies``; forces/stress are derivative outputs w.r.t. positions; cutoff = ``model.r_max``; PBC supported.
Differences: the wrapped network is this package's own :class:`MACE` (the reference wraps ``mace-torch``), and the
dense MATRIX neighbour format is consumed directly by the kernels (a COO list is accepted as well).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.models.mace.model import MACE, MACEConfig


class MACEWrapper(nn.Module, BaseModelMixin):
    def __init__(self, model: MACE | None = None, reconstruction_spec: dict | None = None,
                 neighbor_format: NeighborListFormat = NeighborListFormat.MATRIX, skin: float = 0.0, **config: Any) -> None:
        super().__init__()
        self.model = model if model is not None else MACE(MACEConfig(**config))
        self.reconstruction_spec = reconstruction_spec
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress", "hessian", "atomic_energies"}),
            autograd_outputs=frozenset({"forces", "stress"}), autograd_inputs=frozenset({"positions"}),
            optional_inputs=frozenset({"cell", "pbc", "neighbor_matrix_shifts", "neighbor_list_shifts", "shifts"}),
            supports_pbc=True, needs_pbc=False,
            neighbor_config=NeighborConfig(cutoff=float(self.model.r_max), format=neighbor_format, half_list=False,
                                           skin=skin),
            active_outputs={"energy", "forces"},
        )
        self._csr_cache: tuple[Any, Any] | None = None

    @property
    def embedding_shapes(self) -> dict[str, tuple[int, ...]]:
        return {"node_embeddings": (self.model.hidden_dim(),)}

    def adapt_input(self, data: Any, **kwargs: Any) -> dict[str, Any]:
        pos = data.positions
        n = pos.shape[0]
        if hasattr(data, "num_graphs"):
            batch, ptr, nb = data.batch_idx.long(), data.batch_ptr.long(), data.num_graphs
        else:
            batch = torch.zeros(n, dtype=torch.long, device=pos.device)
            ptr, nb = torch.tensor([0, n], device=pos.device), 1
        cell = getattr(data, "cell", None)
        if cell is not None:
            cell = cell.reshape(nb, 3, 3)
        out: dict[str, Any] = {"positions": pos, "atomic_numbers": data.atomic_numbers, "batch": batch, "ptr": ptr,
                               "cell": cell, "num_graphs": nb, "energy_weights": getattr(data, "energy_weights", None)}
        nm = getattr(data, "neighbor_matrix", None)
        if nm is not None and self.model_config.neighbor_config.format == NeighborListFormat.MATRIX:
            out.update(neighbor_matrix=nm, num_neighbors=data.num_neighbors,
                       neighbor_matrix_shifts=getattr(data, "neighbor_matrix_shifts", None))
            ver = getattr(data, "_neighbor_version", None)
            if ver is not None and pos.is_cuda:
                if self._csr_cache is None or self._csr_cache[0] != ver:
                    from nvalchemi_toolkit_b200.models.mace import native

                    self._csr_cache = (ver, native.build_csr(nm, data.num_neighbors, out["neighbor_matrix_shifts"]))
                out["_csr"] = self._csr_cache[1]
            return out
        nl = getattr(data, "neighbor_list", None)
        if nl is None:
            raise KeyError("MACEWrapper needs neighbour data: run compute_neighbors() or register NeighborListHook")
        valid = (nl < n).all(dim=1)  # sentinel / padding edges are dropped
        nl = nl[valid]
        out["edge_index"] = nl.t().contiguous()
        unit = getattr(data, "neighbor_list_shifts", None)
        if unit is not None and cell is not None:
            unit = unit[valid].to(pos.dtype)
            out["unit_shifts"] = unit
            out["shifts"] = torch.einsum("ei,eij->ej", unit, cell[batch[nl[:, 0]]].to(pos.dtype))
        else:
            sh = getattr(data, "shifts", None)
            out["shifts"] = sh[valid] if sh is not None else pos.new_zeros(nl.shape[0], 3)
        return out

    def forward(self, data: Any, **kwargs: Any) -> dict:
        active = set(self.model_config.active_outputs)
        inputs = self.adapt_input(data)
        res = self.model(inputs, compute_force="forces" in active, compute_stress="stress" in active,
                         compute_hessian="hessian" in active,  # second derivatives run on the differentiable PyTorch path
                         training=self.training)
        res["atomic_energies"] = res.get("node_energy")
        return self.adapt_output(res, data)

    def compute_embeddings(self, data: Any, **kwargs: Any) -> Any:
        inputs = self.adapt_input(data)
        species = self.model.species_index(inputs["atomic_numbers"])
        send, recv, sh = self.model._edges_from(inputs, inputs["positions"], inputs["batch"], inputs["cell"])
        with torch.no_grad():
            _, feats = self.model.node_energies_torch(inputs["positions"], species, send, recv, sh, return_features=True)
        data["node_embeddings"] = torch.cat([f.reshape(f.shape[0], -1) for f in feats[:1]], dim=-1)
        return data

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed import spec as _spec

        if strategy is not None and str(getattr(strategy, "value", strategy)) == "graph_partition":
            return _spec.SPEC_MACE_GRAPH_PARTITION
        return _spec.SPEC_MACE_HALO.with_(message_passes=len(self.model.interactions))

    def checkpoint_spec(self) -> dict:
        from dataclasses import asdict

        return {"cls": "nvalchemi_toolkit_b200.models.mace.MACEWrapper", "config": asdict(self.model.config)}

    def export_model(self, path: Path, as_state_dict: bool = False) -> None:
        payload = self.model.state_dict() if as_state_dict else {"config": self.checkpoint_spec()["config"],
                                                                  "state_dict": self.model.state_dict()}
        torch.save(payload, Path(path))

    @classmethod
    def from_checkpoint(cls, path: str | Path, device: str | torch.device = "cpu", dtype: torch.dtype | None = None,
                        **kwargs: Any) -> "MACEWrapper":
        payload = torch.load(Path(path), map_location=device, weights_only=True)
        model = MACE(MACEConfig(**payload["config"]))
        model.load_state_dict(payload["state_dict"])
        if dtype is not None:
            model = model.to(dtype)
        return cls(model.to(device), reconstruction_spec={"path": str(path)}, **kwargs)
