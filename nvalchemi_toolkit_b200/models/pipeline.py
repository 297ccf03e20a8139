# SPDX-License-Identifier: Apache-2.0
"""Composite models: ``PipelineStep`` / ``PipelineGroup`` / ``PipelineModelWrapper``.

Behaviour follows the reference (``nvalchemi/models/pipeline.py:229-1470``): groups run in declaration order and their
additive outputs (``energy``, ``forces``, ``stress`` by default) are summed; inside a group, steps run in order and an
upstream output can be *wired* onto a batch attribute that a downstream model reads; a group with
``use_autograd=True`` asks its members for energies only, sums them and differentiates once (forces ``-dE/dr``, stress
by the affine strain trick, or a user ``derivative_fn``).  Neighbour data are shared: sub-models whose cutoffs are
within ``max_cutoff_ratio`` of each other use one list built at the largest cutoff, filtered down for the tighter ones.
"""
from __future__ import annotations

import importlib
import json
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch
from torch import nn

from nvalchemi_toolkit_b200 import neighbors as _nb
from nvalchemi_toolkit_b200.models._utils import prepare_strain, sum_outputs
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat

DerivativeFn = Callable[[torch.Tensor, Any, set], dict]


@dataclass
class PipelineStep:
    """A model plus an output→batch-attribute rename map (``{"charges": "node_charges"}``)."""

    model: BaseModelMixin
    wire: dict[str, str] = field(default_factory=dict)


@dataclass
class PipelineGroup:
    steps: list
    use_autograd: bool = False
    derivative_fn: DerivativeFn | None = None


def filter_neighbor_matrix(positions: torch.Tensor, cell: torch.Tensor | None, batch_idx: torch.Tensor,
                           nm: torch.Tensor, num: torch.Tensor, shifts: torch.Tensor | None, cutoff: float
                           ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """Rows of a dense neighbour matrix restricted to pairs closer than ``cutoff`` (kept entries stay left-packed).
    Reference: ``nvalchemi/models/_ops/neighbor_filter.py:43-430``."""
    n, k = nm.shape
    valid = torch.arange(k, device=nm.device)[None] < num[:, None].clamp_max(k)
    j = nm.long().clamp_max(max(n - 1, 0))
    d = positions.detach()[j] - positions.detach()[:, None, :]
    if shifts is not None and cell is not None:
        d = d + torch.einsum("nki,nij->nkj", shifts.to(d.dtype), cell.to(d.dtype)[batch_idx.long()])
    keep = valid & (d.pow(2).sum(-1) < cutoff * cutoff)
    order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)
    new_num = keep.sum(1).to(num.dtype)
    packed = torch.arange(k, device=nm.device)[None] < new_num[:, None]
    new_nm = torch.where(packed, torch.gather(nm, 1, order), torch.full_like(nm, n))
    new_sh = None
    if shifts is not None:
        new_sh = torch.gather(shifts, 1, order[..., None].expand(-1, -1, 3)) * packed[..., None].to(shifts.dtype)
    return new_nm, new_num, new_sh


def _put(data: Any, key: str, value: torch.Tensor) -> None:
    """Attach a tensor to the batch, registering its level from its leading dimension when the key is new."""
    try:
        data[key] = value
    except KeyError:
        level = "node" if value.shape[0] == data.num_nodes else "system"
        data.add_key(key, value, level=level, overwrite=True)


@dataclass
class _Source:
    cutoff: float
    half_list: bool
    hook: Any = None


class _PipelineNeighborHook:
    """Runs one ``NeighborListHook`` per neighbour source and parks each result on the batch."""

    frequency = 1

    def __init__(self, sources: list[_Source], stage: Any) -> None:
        self.sources, self.stage = sources, stage

    def __call__(self, ctx: Any, stage: Any) -> None:
        batch = ctx.batch
        store = {}
        for sid, src in enumerate(self.sources):
            src.hook(ctx, stage)
            nm, num, sh = src.hook._bufs
            store[sid] = (nm, num, sh, src.hook.config.cutoff + src.hook.skin, (id(src.hook), src.hook.version))
        object.__setattr__(batch, "_pipeline_neighbors", store)


class PipelineModelWrapper(nn.Module, BaseModelMixin):
    def __init__(self, groups: list[PipelineGroup], additive_keys: set[str] | None = None, *,
                 neighbor_adaptation: str = "auto", max_cutoff_ratio: float = 1.5) -> None:
        super().__init__()
        if neighbor_adaptation not in ("auto", "always", "never"):
            raise ValueError("PipelineModelWrapper: neighbor_adaptation must be one of 'auto', 'always', or 'never'.")
        if max_cutoff_ratio < 1.0:
            raise ValueError("PipelineModelWrapper: max_cutoff_ratio must be >= 1.0.")
        self._adaptation, self._ratio = neighbor_adaptation, float(max_cutoff_ratio)
        self.groups: list[PipelineGroup] = []
        for g in groups:
            steps = [s if isinstance(s, PipelineStep) else PipelineStep(model=s) for s in g.steps]
            self.groups.append(PipelineGroup(steps=steps, use_autograd=g.use_autograd, derivative_fn=g.derivative_fn))
        self._models = nn.ModuleList(s.model for g in self.groups for s in g.steps)
        self.additive_keys = set(additive_keys or {"energy", "forces", "stress"})
        batch_required = self._check_wiring()
        self._plan_neighbors()
        self.model_config = self._build_config(batch_required)
        self._configure_sub_models()

    # ---- construction ----------------------------------------------------------
    def _steps(self) -> list[PipelineStep]:
        return [s for g in self.groups for s in g.steps]

    def _check_wiring(self) -> set[str]:
        """Inputs no upstream step provides must come from the batch; a wire must name an output its model has."""
        provided: set[str] = set()
        required: set[str] = set()
        for step in self._steps():
            cfg = step.model.model_config
            for out_key in step.wire:
                if out_key not in cfg.outputs:
                    raise ValueError(f"wire source '{out_key}' is not an output of {type(step.model).__name__} "
                                     f"(outputs: {sorted(cfg.outputs)})")
            required |= {k for k in cfg.required_inputs if k not in provided}
            provided |= set(step.wire.values()) | (set(cfg.outputs) - set(step.wire))
        return required

    def _plan_neighbors(self) -> None:
        """Cluster sub-model cutoffs (per half/full list kind) into shared sources."""
        self._sources: list[_Source] = []
        self._step_source: dict[int, tuple[int, float]] = {}
        by_kind: dict[bool, list[tuple[float, int]]] = {}
        for idx, step in enumerate(self._steps()):
            nc = step.model.model_config.neighbor_config
            if nc is not None:
                by_kind.setdefault(bool(nc.half_list), []).append((float(nc.cutoff), idx))
        for half, items in by_kind.items():
            items.sort(reverse=True)
            current: _Source | None = None
            for cutoff, idx in items:
                share = current is not None and (
                    self._adaptation == "always" or
                    (self._adaptation == "auto" and current.cutoff <= self._ratio * cutoff) or
                    (self._adaptation == "never" and current.cutoff == cutoff))
                if not share:
                    current = _Source(cutoff=cutoff, half_list=half)
                    self._sources.append(current)
                self._step_source[idx] = (len(self._sources) - 1, cutoff)

    def _build_config(self, batch_required: set[str]) -> ModelConfig:
        cfgs = [s.model.model_config for s in self._steps()]
        outputs: set[str] = set().union(*[set(c.outputs) for c in cfgs])
        active: set[str] = set().union(*[set(c.active_outputs) for c in cfgs])
        auto_groups = [g for g in self.groups if g.use_autograd]
        autograd_outputs: set[str] = set()
        if auto_groups:
            autograd_outputs = {"forces", "stress"}
            outputs |= autograd_outputs
        else:
            autograd_outputs = set().union(*[set(c.autograd_outputs) for c in cfgs])
        cut = max((s.cutoff for s in self._sources), default=None)
        nc = None
        if cut is not None:
            skin = max((c.neighbor_config.skin for c in cfgs if c.neighbor_config is not None), default=0.0)
            nc = NeighborConfig(cutoff=cut, format=NeighborListFormat.MATRIX, half_list=False, skin=skin)
        return ModelConfig(outputs=frozenset(outputs), autograd_outputs=frozenset(autograd_outputs),
                           autograd_inputs=frozenset({"positions"}) if autograd_outputs else frozenset(),
                           required_inputs=frozenset(batch_required),
                           optional_inputs=frozenset().union(*[c.optional_inputs for c in cfgs]),
                           supports_pbc=all(c.supports_pbc for c in cfgs), needs_pbc=any(c.needs_pbc for c in cfgs),
                           neighbor_config=nc, active_outputs=active & outputs)

    def _configure_sub_models(self) -> None:
        """Members of autograd groups produce energies (and wired quantities) only."""
        for g in self.groups:
            if not g.use_autograd:
                continue
            for s in g.steps:
                cfg = s.model.model_config
                keep = {"energy"} | set(s.wire) | (set(cfg.active_outputs) - {"forces", "stress", "virial", "hessian"})
                cfg.active_outputs = keep & set(cfg.outputs)

    @property
    def embedding_shapes(self) -> dict[str, tuple[int, ...]]:
        out: dict[str, tuple[int, ...]] = {}
        for s in self._steps():
            try:
                out.update(s.model.embedding_shapes)
            except NotImplementedError:
                pass
        return out

    def compute_embeddings(self, data: Any, **kwargs: Any) -> Any:
        for s in self._steps():
            try:
                data = s.model.compute_embeddings(data, **kwargs)
            except NotImplementedError:
                continue
        return data

    def extra_repr(self) -> str:
        return ", ".join(f"group{i}[{'autograd' if g.use_autograd else 'direct'}]=" +
                         "+".join(type(s.model).__name__ for s in g.steps) for i, g in enumerate(self.groups))

    # ---- neighbours ------------------------------------------------------------
    def make_neighbor_hooks(self, max_neighbors: int | None = None, neighbor_list_method: str | None = None) -> list:
        from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage
        from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook

        if not self._sources:
            return []
        skin = self.model_config.neighbor_config.skin
        for src in self._sources:
            src.hook = NeighborListHook(NeighborConfig(cutoff=src.cutoff, format=NeighborListFormat.MATRIX,
                                                       half_list=src.half_list, skin=skin), skin=skin,
                                        max_neighbors=max_neighbors, method=neighbor_list_method,
                                        stage=DynamicsStage.BEFORE_COMPUTE)
        return [_PipelineNeighborHook(self._sources, DynamicsStage.BEFORE_COMPUTE)]

    def _select_neighbors(self, data: Any, step_idx: int, model: BaseModelMixin) -> None:
        plan = self._step_source.get(step_idx)
        if plan is None:
            return
        store = getattr(data, "_pipeline_neighbors", None)
        if store is None:
            return  # the caller supplied neighbour data directly (single list for every member)
        sid, cutoff = plan
        nm, num, sh, src_cut, version = store[sid]
        nc = model.model_config.neighbor_config
        if src_cut > cutoff * (1.0 + 1e-9) and self._adaptation != "never":
            cell = getattr(data, "cell", None)
            nm, num, sh = filter_neighbor_matrix(data.positions, cell.reshape(-1, 3, 3) if cell is not None else None,
                                                 data.batch_idx, nm, num, sh, cutoff + nc.skin)
        _nb.write_neighbor_data_to_batch(data, nm, num, sh, nc.format, cutoff)
        object.__setattr__(data, "_neighbor_version", (version, step_idx))

    # ---- forward ---------------------------------------------------------------
    def _call_step(self, step: PipelineStep, step_idx: int, data: Any, **kwargs: Any) -> dict:
        self._select_neighbors(data, step_idx, step.model)
        out = step.model(data, **kwargs)
        for out_key, attr in step.wire.items():
            value = out.get(out_key)
            if value is None:
                raise RuntimeError(f"{type(step.model).__name__} did not produce '{out_key}' needed by wire → '{attr}'")
            _put(data, attr, value)
        for key, value in out.items():  # auto-wiring: outputs a downstream member declares as a required input
            if value is not None and key not in step.wire and key in self._downstream_inputs(step_idx):
                _put(data, key, value)
        return out

    def _downstream_inputs(self, step_idx: int) -> set[str]:
        later = self._steps()[step_idx + 1:]
        return set().union(*[set(s.model.model_config.required_inputs) for s in later]) if later else set()

    def forward(self, data: Any, **kwargs: Any) -> "OrderedDict[str, torch.Tensor | None]":
        active = set(self.model_config.active_outputs)
        results = []
        idx = 0
        for g in self.groups:
            if g.use_autograd:
                results.append(self._run_autograd_group(g, idx, data, active, **kwargs))
            else:
                outs = []
                for k, s in enumerate(g.steps):
                    outs.append({k2: v for k2, v in self._call_step(s, idx + k, data, **kwargs).items()})
                results.append(sum_outputs(*outs, additive_keys=frozenset(self.additive_keys)))
            idx += len(g.steps)
        total = sum_outputs(*results, additive_keys=frozenset(self.additive_keys))
        return self.adapt_output(total, data)

    def _run_autograd_group(self, g: PipelineGroup, first_idx: int, data: Any, active: set, **kwargs: Any) -> dict:
        requested = {k for k in ("forces", "stress") if k in active}
        pos0, cell0 = data.positions, getattr(data, "cell", None)
        batch_idx = data.batch_idx if hasattr(data, "batch_idx") else torch.zeros(pos0.shape[0], dtype=torch.long,
                                                                                   device=pos0.device)
        with torch.enable_grad():
            leaf = pos0.detach().requires_grad_(True)
            strain = None
            if "stress" in requested and cell0 is not None:
                spos, scell, strain = prepare_strain(leaf, cell0.detach().reshape(-1, 3, 3), batch_idx)
                data["positions"], data["cell"] = spos, scell.reshape(cell0.shape)
            else:
                data["positions"] = leaf
            try:
                outs = [self._call_step(s, first_idx + k, data, **kwargs) for k, s in enumerate(g.steps)]
                summed = sum_outputs(*outs, additive_keys=frozenset({"energy"}))
                energy = summed["energy"]
                if g.derivative_fn is not None:
                    object.__setattr__(data, "_pipeline_leaves", {"positions": leaf, "strain": strain})
                    summed.update(g.derivative_fn(energy, data, requested))
                elif requested:
                    summed.update(self._default_derivatives(energy, leaf, strain, cell0, requested))
            finally:
                data["positions"] = pos0
                if strain is not None:
                    data["cell"] = cell0
        if not self.training:
            summed = {k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in summed.items()}
        return summed

    def _default_derivatives(self, energy: torch.Tensor, leaf: torch.Tensor, strain: torch.Tensor | None,
                             cell: torch.Tensor | None, requested: set) -> dict:
        wrt = [leaf] + ([strain] if strain is not None else [])
        grads = torch.autograd.grad(energy.sum(), wrt, create_graph=self.training, retain_graph=self.training,
                                    allow_unused=True)
        out: dict[str, torch.Tensor] = {}
        if "forces" in requested:
            out["forces"] = -grads[0] if grads[0] is not None else torch.zeros_like(leaf)
        if "stress" in requested and strain is not None:
            vol = torch.linalg.det(cell.detach().reshape(-1, 3, 3)).abs().clamp_min(1e-30)
            gs = grads[1] if grads[1] is not None else torch.zeros_like(strain)
            out["stress"] = gs / vol[:, None, None]
        return out

    # ---- persistence -------------------------------------------------------------
    def export_model(self, path: Path, as_state_dict: bool = False) -> None:
        if as_state_dict:
            torch.save(self.state_dict(), Path(path))
        else:
            self.save(path)

    def save(self, path: str | Path) -> None:
        """One file: the group layout, each member's ``checkpoint_spec()`` and its weights."""
        layout = []
        for g in self.groups:
            members = []
            for s in g.steps:
                spec_fn = getattr(s.model, "checkpoint_spec", None)
                if spec_fn is None:
                    raise TypeError(f"{type(s.model).__name__} has no checkpoint_spec(); it cannot be saved in a pipeline")
                members.append({"spec": spec_fn(), "wire": s.wire,
                                "active_outputs": sorted(s.model.model_config.active_outputs)})
            if g.derivative_fn is not None:
                raise TypeError("a pipeline with a custom derivative_fn cannot be serialised")
            layout.append({"use_autograd": g.use_autograd, "steps": members})
        payload = {"layout": json.dumps(layout), "additive_keys": sorted(self.additive_keys),
                   "neighbor_adaptation": self._adaptation, "max_cutoff_ratio": self._ratio,
                   "active_outputs": sorted(self.model_config.active_outputs),
                   "state": [s.model.state_dict() for s in self._steps()]}
        torch.save(payload, Path(path))

    @classmethod
    def load(cls, path: str | Path, device: str | torch.device = "cpu") -> "PipelineModelWrapper":
        payload = torch.load(Path(path), map_location=device, weights_only=True)
        groups, flat = [], []
        for g in json.loads(payload["layout"]):
            steps = []
            for m in g["steps"]:
                module, _, name = m["spec"]["cls"].rpartition(".")
                klass = getattr(importlib.import_module(module), name)
                model = klass(**m["spec"].get("config", {})) if not hasattr(klass, "from_spec") else klass.from_spec(m["spec"])
                model.model_config.active_outputs = set(m["active_outputs"])
                steps.append(PipelineStep(model=model, wire=dict(m["wire"])))
                flat.append(model)
            groups.append(PipelineGroup(steps=steps, use_autograd=g["use_autograd"]))
        for model, state in zip(flat, payload["state"]):
            model.load_state_dict(state)
            model.to(device)
        pipe = cls(groups, set(payload["additive_keys"]), neighbor_adaptation=payload["neighbor_adaptation"],
                   max_cutoff_ratio=payload["max_cutoff_ratio"])
        pipe.model_config.active_outputs = set(payload["active_outputs"])
        return pipe
