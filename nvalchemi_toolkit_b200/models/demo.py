# SPDX-License-Identifier: Apache-2.0
"""Small non-periodic demo potential used for plumbing tests and examples.

Architecture as described for the reference's ``DemoModel`` (``nvalchemi/models/demo.py:36-325``):
an atomic-number embedding ``Embedding(100, H, padding_idx=0, max_norm=1)``, a coordinate branch
``Linear(3,H) + LayerNorm + SiLU``, a joint MLP, and a per-atom energy projection summed per graph;
forces are ``-dE/dr`` by autograd.  The model is not physical (it is not translation invariant); it
exists to exercise the data, dynamics and hook layers cheaply on CPU and GPU.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig


class DemoModel(nn.Module):
    def __init__(self, hidden_dim: int = 64) -> None:
        super().__init__()
        self.hidden_dim = hidden_dim
        self.embedding = nn.Embedding(100, hidden_dim, padding_idx=0, max_norm=1.0)
        self.coord_embedding = nn.Sequential(nn.Linear(3, hidden_dim, bias=False), nn.LayerNorm(hidden_dim), nn.SiLU())
        self.joint_mlp = nn.Sequential(nn.Linear(2 * hidden_dim, hidden_dim), nn.LayerNorm(hidden_dim), nn.SiLU(),
                                       nn.Linear(hidden_dim, hidden_dim), nn.LayerNorm(hidden_dim), nn.SiLU())
        self.projection = nn.Linear(hidden_dim, 1, bias=False)

    def node_embeddings(self, atomic_numbers: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        z = self.embedding(atomic_numbers.long())
        c = self.coord_embedding(positions)
        return self.joint_mlp(torch.cat([z, c], dim=-1))

    def forward(self, atomic_numbers: torch.Tensor, positions: torch.Tensor, batch_idx: torch.Tensor,
                num_graphs: int) -> tuple[torch.Tensor, torch.Tensor]:
        h = self.node_embeddings(atomic_numbers, positions)
        node_e = self.projection(h)
        energy = torch.zeros(num_graphs, 1, dtype=node_e.dtype, device=node_e.device)
        energy.index_add_(0, batch_idx.long(), node_e)
        return energy, h


class DemoModelWrapper(nn.Module, BaseModelMixin):
    """``BaseModelMixin`` adapter around :class:`DemoModel` (energy, autograd forces, embeddings)."""

    def __init__(self, model: DemoModel | None = None, hidden_dim: int = 64) -> None:
        super().__init__()
        self.model = model if model is not None else DemoModel(hidden_dim)
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces"}), autograd_outputs=frozenset({"forces"}),
            autograd_inputs=frozenset({"positions"}), supports_pbc=False, needs_pbc=False, neighbor_config=None,
        )

    @property
    def embedding_shapes(self) -> dict[str, tuple[int, ...]]:
        h = self.model.hidden_dim
        return {"node_embeddings": (h,), "graph_embeddings": (h,)}

    def compute_embeddings(self, data: Any, **kwargs: Any) -> Any:
        with torch.no_grad():
            batch_idx, nb = self._graph_index(data)
            h = self.model.node_embeddings(data.atomic_numbers, data.positions)
            g = torch.zeros(nb, h.shape[-1], dtype=h.dtype, device=h.device).index_add_(0, batch_idx.long(), h)
        data["node_embeddings"] = h
        data["graph_embeddings"] = g
        return data

    @staticmethod
    def _graph_index(data: Any) -> tuple[torch.Tensor, int]:
        if hasattr(data, "num_graphs"):
            return data.batch_idx, data.num_graphs
        n = data.positions.shape[0]
        return torch.zeros(n, dtype=torch.int32, device=data.positions.device), 1

    def forward(self, data: Any, **kwargs: Any) -> dict:
        want_forces = "forces" in self.model_config.active_outputs
        inputs = self.adapt_input(data)
        pos = inputs["positions"]
        batch_idx, nb = self._graph_index(data)
        with torch.enable_grad():
            if want_forces and not pos.requires_grad:
                pos.requires_grad_(True)
            energy, _ = self.model(inputs["atomic_numbers"], pos, batch_idx, nb)
            out = {"energy": energy}
            if want_forces:
                (g,) = torch.autograd.grad(energy.sum(), pos, create_graph=self.training)
                out["forces"] = -g
        return self.adapt_output(out, data)

    def checkpoint_spec(self) -> dict:
        return {"cls": "nvalchemi_toolkit_b200.models.demo.DemoModelWrapper", "config": {"hidden_dim": self.model.hidden_dim}}

    def distribution_spec(self, strategy: Any = None) -> Any:
        from nvalchemi_toolkit_b200.distributed.spec import SPEC_DEMO

        return SPEC_DEMO

    def export_model(self, path: Any, as_state_dict: bool = False) -> None:
        torch.save(self.model.state_dict() if as_state_dict else self.model, path)
