# SPDX-License-Identifier: Apache-2.0
"""Model contract: ``ModelConfig`` capabilities + ``BaseModelMixin`` adapters.

API parity target: reference ``nvalchemi/models/base.py:38-734``.  A wrapper sets
``self.model_config`` in ``__init__`` (checked by ``__init_subclass__``), reads its
inputs from a ``Batch`` via ``adapt_input`` and returns canonical keys
(``energy [B,1]``, ``forces [V,3]``, ``stress [B,3,3]`` ...) via ``adapt_output``.
"""
from __future__ import annotations

import abc
import functools
import warnings
from collections import OrderedDict
from enum import Enum
from pathlib import Path
from typing import Any

import torch
from pydantic import BaseModel, ConfigDict, Field, model_validator


class NeighborListFormat(str, Enum):
    """``COO``: ``neighbor_list [E,2]`` (source, target); ``MATRIX``: ``neighbor_matrix [V,K]`` + ``num_neighbors``."""

    COO = "coo"
    MATRIX = "matrix"


class NeighborConfig(BaseModel):
    cutoff: float
    format: NeighborListFormat = NeighborListFormat.COO
    half_list: bool = False
    skin: float = 0.0


class ModelConfig(BaseModel):
    """Frozen capability fields plus mutable runtime fields (``active_outputs``, ``gradient_keys``)."""

    model_config = ConfigDict(validate_assignment=True)

    outputs: frozenset[str] = Field(default_factory=lambda: frozenset({"energy"}))
    autograd_outputs: frozenset[str] = Field(default_factory=frozenset)
    autograd_inputs: frozenset[str] = Field(default_factory=frozenset)
    required_inputs: frozenset[str] = Field(default_factory=frozenset)
    optional_inputs: frozenset[str] = Field(default_factory=frozenset)
    supports_pbc: bool = False
    needs_pbc: bool = False
    neighbor_config: NeighborConfig | None = None
    active_outputs: set[str] | None = None
    gradient_keys: set[str] = Field(default_factory=set)

    @model_validator(mode="after")
    def _default_active_outputs(self) -> "ModelConfig":
        if self.active_outputs is None:
            self.__dict__["active_outputs"] = set(self.outputs)
        return self

    @property
    def needs_neighborlist(self) -> bool:
        return self.neighbor_config is not None


class BaseModelMixin(abc.ABC):
    """Mixin for ``nn.Module`` wrappers that plug into dynamics, training and distribution."""

    _dist_ctx: Any = None

    def __init_subclass__(cls, **kwargs: Any) -> None:
        super().__init_subclass__(**kwargs)
        if "extra_repr" not in cls.__dict__:
            cls.extra_repr = BaseModelMixin._config_extra_repr  # type: ignore[assignment]
        if "__init__" in cls.__dict__:
            original = cls.__init__

            @functools.wraps(original)
            def _checked(self: Any, *a: Any, **k: Any) -> None:
                original(self, *a, **k)
                if type(self).__init__ is _checked and not hasattr(self, "model_config"):
                    raise TypeError(
                        f"{type(self).__name__}.__init__() must set self.model_config = ModelConfig(...)."
                    )

            cls.__init__ = _checked  # type: ignore[assignment]

    def _config_extra_repr(self: Any) -> str:
        cfg = getattr(self, "model_config", None)
        if cfg is None:
            return "model_config=<not set>"
        parts = [f"outputs={{{', '.join(sorted(cfg.outputs))}}}"]
        if set(cfg.active_outputs) != set(cfg.outputs):
            parts.append(f"active_outputs={{{', '.join(sorted(cfg.active_outputs))}}}")
        if cfg.autograd_outputs:
            parts.append(f"autograd_outputs={{{', '.join(sorted(cfg.autograd_outputs))}}}")
        if cfg.neighbor_config is not None:
            nc = cfg.neighbor_config
            parts.append(f"neighbors=(cutoff={nc.cutoff}, format={nc.format.value}"
                         + (", half_list" if nc.half_list else "") + ")")
        return "\n".join(parts)

    # -- embeddings ----------------------------------------------------------
    @property
    def embedding_shapes(self) -> dict[str, tuple[int, ...]]:
        return {}

    def compute_embeddings(self, data: Any, **kwargs: Any) -> Any:
        raise NotImplementedError(f"{type(self).__name__} does not expose embeddings")

    def direct_derivative_keys(self) -> set[str]:
        return set()

    def set_config(self, key: str, value: Any) -> None:
        if key not in type(self.model_config).model_fields:
            raise AttributeError(
                f"ModelConfig has no field '{key}'.  Available fields: {list(type(self.model_config).model_fields)}"
            )
        setattr(self.model_config, key, value)

    # -- IO adapters -----------------------------------------------------------
    def input_data(self) -> set[str]:
        base = {"positions", "atomic_numbers"}
        nc = self.model_config.neighbor_config
        if nc is not None:
            if nc.format == NeighborListFormat.COO:
                base.add("neighbor_list")
            else:
                base |= {"neighbor_matrix", "num_neighbors"}
        if self.model_config.needs_pbc:
            base.add("pbc")
        return base | set(self.model_config.required_inputs)

    def output_data(self) -> set[str]:
        active, supported = set(self.model_config.active_outputs), set(self.model_config.outputs)
        if active - supported:
            warnings.warn(f"Requested {active - supported} but model only supports {supported}.", UserWarning,
                          stacklevel=2)
        return active & supported

    def adapt_input(self, data: Any, **kwargs: Any) -> dict[str, Any]:
        cfg = self.model_config
        grad_keys = set(cfg.gradient_keys)
        if cfg.autograd_outputs & set(cfg.active_outputs):
            grad_keys |= cfg.autograd_inputs
        for key in grad_keys:
            value = getattr(data, key, None)
            if value is None:
                raise KeyError(f"'{key}' required for gradient computation, but not found in batch.")
            if not isinstance(value, torch.Tensor):
                raise TypeError(f"'{key}' set to require gradients, but is {type(value)} (not a tensor).")
            value.requires_grad_(True)
        out: dict[str, Any] = {}
        for key in self.input_data():
            value = getattr(data, key, None)
            if value is None:
                raise KeyError(f"'{key}' required but not found in input data.")
            out[key] = value
        for key in cfg.optional_inputs:
            value = getattr(data, key, None)
            if value is not None:
                out[key] = value
        return out

    def adapt_output(self, model_output: Any, data: Any) -> "OrderedDict[str, torch.Tensor | None]":
        output: OrderedDict[str, torch.Tensor | None] = OrderedDict((k, None) for k in sorted(self.output_data()))
        if isinstance(model_output, dict):
            for key in output:
                value = model_output.get(key)
                if value is not None:
                    if key == "energy" and value.ndim == 1:
                        value = value.unsqueeze(-1)
                    output[key] = value
        return output

    def add_output_head(self, prefix: str) -> None:
        raise NotImplementedError

    # -- distribution seams ---------------------------------------------------
    def distribution_spec(self, strategy: Any = None) -> Any:
        return None

    def distributed_setup(self, ctx: Any) -> None:
        self._dist_ctx = ctx

    def distributed_teardown(self) -> None:
        self._dist_ctx = None

    def export_model(self, path: Path, as_state_dict: bool = False) -> None:
        if isinstance(self, torch.nn.Module) and as_state_dict:
            torch.save(self.state_dict(), Path(path))
            return
        raise NotImplementedError

    def __add__(self, other: "BaseModelMixin") -> Any:
        from nvalchemi_toolkit_b200.models.pipeline import PipelineGroup, PipelineModelWrapper

        if isinstance(self, PipelineModelWrapper):
            return PipelineModelWrapper(groups=list(self.groups) + [PipelineGroup(steps=[other])])
        return PipelineModelWrapper(groups=[PipelineGroup(steps=[self]), PipelineGroup(steps=[other])])

    def make_neighbor_hooks(self, max_neighbors: int | None = None, neighbor_list_method: str | None = None) -> list:
        from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage
        from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook

        nc = self.model_config.neighbor_config
        if nc is None:
            return []
        return [NeighborListHook(nc, skin=nc.skin, max_neighbors=max_neighbors, method=neighbor_list_method,
                                 stage=DynamicsStage.BEFORE_COMPUTE)]
