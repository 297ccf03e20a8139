# SPDX-License-Identifier: Apache-2.0
"""Adapter for AIMNet2 models (optional dependency ``aimnet``).

Reference: ``nvalchemi/models/aimnet2.py:93-822``: the wrapped network consumes a padded dictionary (``coord``,
``numbers``, ``charge``, ``mol_idx``, ``nbmat`` with one trailing padding atom) and returns ``energy`` and ``charges``;
forces and stresses follow from autograd (strain trick), its internal Coulomb and dispersion heads are switched off so
that long-range terms are composed explicitly (``AIMNet2Wrapper + PMEModelWrapper + DFTD3ModelWrapper`` with a wire
``{"charges": "node_charges"}``).  The adapter accepts any ``nn.Module`` with that calling convention; loading named
checkpoints needs the ``aimnet`` package.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from nvalchemi_toolkit_b200._optional import OptionalDependency
from nvalchemi_toolkit_b200.models._utils import prepare_strain
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat


class AIMNet2Wrapper(nn.Module, BaseModelMixin):
    def __init__(self, model: nn.Module, cutoff: float | None = None, embedding_dim: int | None = None) -> None:
        super().__init__()
        self.model = model
        self.cutoff = float(cutoff if cutoff is not None else getattr(model, "cutoff", 5.0))
        self._embedding_dim = embedding_dim
        for name in ("lrcoulomb", "srcoulomb", "dftd3", "d3bj"):  # long-range heads are composed outside
            head = getattr(getattr(model, "outputs", None), name, None)
            if head is not None and hasattr(head, "enabled"):
                head.enabled = False
        self.model_config = ModelConfig(
            outputs=frozenset({"energy", "forces", "stress", "charges", "node_embeddings"}),
            autograd_outputs=frozenset({"forces", "stress"}), autograd_inputs=frozenset({"positions"}),
            optional_inputs=frozenset({"cell", "pbc", "charge", "neighbor_matrix_shifts"}), supports_pbc=True,
            neighbor_config=NeighborConfig(cutoff=self.cutoff, format=NeighborListFormat.MATRIX, half_list=False),
            active_outputs={"energy", "forces", "charges"})

    @classmethod
    def from_checkpoint(cls, name_or_path: str, device: str | torch.device = "cpu", **kw: Any) -> "AIMNet2Wrapper":
        aimnet = OptionalDependency.AIMNET.import_module()
        calc = aimnet.calculators.AIMNet2Calculator(name_or_path)
        return cls(calc.model.to(device), cutoff=float(getattr(calc, "cutoff", 5.0)), **kw)

    @property
    def embedding_shapes(self) -> dict[str, tuple[int, ...]]:
        return {"node_embeddings": (self._embedding_dim or 256,)}

    def adapt_input(self, data: Any, **kwargs: Any) -> dict[str, Any]:
        pos = data.positions
        n, dev = pos.shape[0], pos.device
        nb = data.num_graphs if hasattr(data, "num_graphs") else 1
        mol_idx = data.batch_idx.long() if hasattr(data, "batch_idx") else torch.zeros(n, dtype=torch.long, device=dev)
        nm = data.neighbor_matrix.long()
        k = nm.shape[1]
        valid = torch.arange(k, device=dev)[None] < data.num_neighbors[:, None]
        nbmat = torch.where(valid, nm, torch.full_like(nm, n))          # padding index n
        nbmat = torch.cat([nbmat, torch.full((1, k), n, dtype=torch.long, device=dev)])
        charge = getattr(data, "charge", None)
        out = {"coord": torch.cat([pos, pos.new_zeros(1, 3)]),
               "numbers": torch.cat([data.atomic_numbers.long(), data.atomic_numbers.new_zeros(1).long()]),
               "mol_idx": torch.cat([mol_idx, mol_idx.new_full((1,), max(nb - 1, 0))]),
               "charge": charge.reshape(nb).to(pos.dtype) if charge is not None else pos.new_zeros(nb), "nbmat": nbmat}
        sh = getattr(data, "neighbor_matrix_shifts", None)
        cell = getattr(data, "cell", None)
        if sh is not None and cell is not None:
            cells = cell.reshape(nb, 3, 3)
            shifts = torch.einsum("nki,nij->nkj", sh.to(pos.dtype), cells[mol_idx]) * valid[..., None]
            out["shifts"] = torch.cat([shifts, shifts.new_zeros(1, k, 3)])
            out["cell"] = cells
        return out

    def forward(self, data: Any, **kwargs: Any) -> dict:
        active = set(self.model_config.active_outputs)
        want_f, want_s = "forces" in active, "stress" in active
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
            out: dict[str, Any] = {"energy": energy, "charges": res.get("charges", None)}
            if out["charges"] is not None:
                out["charges"] = out["charges"][: pos0.shape[0]]
            aim = res.get("aim")
            if aim is not None:
                out["node_embeddings"] = aim[: pos0.shape[0]]
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
        from nvalchemi_toolkit_b200.distributed import spec as _spec

        if strategy is not None and str(getattr(strategy, "value", strategy)) == "graph_partition":
            return _spec.SPEC_AIMNET2_GRAPH_PARTITION
        return _spec.SPEC_AIMNET2_HALO
