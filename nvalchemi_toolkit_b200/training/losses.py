# SPDX-License-Identifier: Apache-2.0
"""Loss terms, weight schedules and their composition.

Reference: ``nvalchemi/training/losses/{composition,terms,reductions,schedules}.py``.  A term compares
``predictions[prediction_key]`` with ``batch[target_key]``; terms compose with ``+`` and ``*`` into a
``ComposedLossFunction`` whose call returns ``{"total_loss": ..., "<name>": ...}``.  Weights may be constants or
schedules evaluated at ``(step, epoch)``.  Per-atom quantities are first reduced per graph (sum or mean over the graph's
atoms) so large systems do not dominate a batch."""
from __future__ import annotations

import math
from typing import Any, Callable

import torch



# ------------------------------------------------------------------ schedules
class LossWeightSchedule:
    def __call__(self, step: int, epoch: int = 0) -> float:  # pragma: no cover - interface
        raise NotImplementedError

    def to_spec(self) -> dict[str, Any]:
        return {"cls": type(self).__name__, **{k: v for k, v in self.__dict__.items()}}


class ConstantWeight(LossWeightSchedule):
    def __init__(self, value: float) -> None:
        self.value = float(value)

    def __call__(self, step: int, epoch: int = 0) -> float:
        return self.value


class LinearWeight(LossWeightSchedule):
    def __init__(self, start: float, end: float, num_steps: int, per_epoch: bool = False) -> None:
        self.start, self.end, self.num_steps, self.per_epoch = float(start), float(end), int(num_steps), per_epoch

    def __call__(self, step: int, epoch: int = 0) -> float:
        t = min((epoch if self.per_epoch else step) / max(self.num_steps, 1), 1.0)
        return self.start + (self.end - self.start) * t


class CosineWeight(LinearWeight):
    def __call__(self, step: int, epoch: int = 0) -> float:
        t = min((epoch if self.per_epoch else step) / max(self.num_steps, 1), 1.0)
        return self.end + 0.5 * (self.start - self.end) * (1.0 + math.cos(math.pi * t))


class PiecewiseWeight(LossWeightSchedule):
    def __init__(self, boundaries: list[int], values: list[float], per_epoch: bool = False) -> None:
        if len(values) != len(boundaries) + 1:
            raise ValueError("PiecewiseWeight needs len(values) == len(boundaries) + 1")
        self.boundaries, self.values, self.per_epoch = list(boundaries), [float(v) for v in values], per_epoch

    def __call__(self, step: int, epoch: int = 0) -> float:
        x = epoch if self.per_epoch else step
        return self.values[sum(1 for b in self.boundaries if x >= b)]


_SCHEDULES = {c.__name__: c for c in (ConstantWeight, LinearWeight, CosineWeight, PiecewiseWeight)}


def schedule_from_spec(spec: Any) -> "LossWeightSchedule | float":
    if isinstance(spec, dict) and "cls" in spec:
        kw = {k: v for k, v in spec.items() if k != "cls"}
        return _SCHEDULES[spec["cls"]](**kw)
    return spec


# ------------------------------------------------------------------ reductions
def per_graph_sum(values: torch.Tensor, batch_idx: torch.Tensor, num_graphs: int) -> torch.Tensor:
    flat = values.reshape(values.shape[0], -1).sum(-1)
    return torch.zeros(num_graphs, dtype=values.dtype, device=values.device).index_add_(0, batch_idx.long(), flat)


def per_graph_mean(values: torch.Tensor, batch_idx: torch.Tensor, num_graphs: int) -> torch.Tensor:
    cnt = torch.bincount(batch_idx.long(), minlength=num_graphs).clamp_min(1).to(values.dtype)
    width = values.reshape(values.shape[0], -1).shape[1]
    return per_graph_sum(values, batch_idx, num_graphs) / (cnt * width)


def frobenius_mse(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return ((pred - target) ** 2).reshape(pred.shape[0], -1).mean(-1)


# ------------------------------------------------------------------ terms
class BaseLossFunction:
    """One weighted term.  Subclasses implement ``per_graph(pred, target, batch) -> [B]``."""

    default_key = "energy"

    def __init__(self, target_key: str | None = None, prediction_key: str | None = None, weight: Any = 1.0,
                 name: str | None = None, dtype: torch.dtype | None = None) -> None:
        self.target_key = target_key or self.default_key
        self.prediction_key = prediction_key or self.target_key
        self.weight = weight
        self.name = name or f"{type(self).__name__}[{self.prediction_key}]"
        self.dtype = dtype

    def weight_at(self, step: int, epoch: int) -> float:
        return float(self.weight(step, epoch)) if callable(self.weight) else float(self.weight)

    def per_graph(self, pred: torch.Tensor, target: torch.Tensor, batch: Any) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def __call__(self, predictions: dict, batch: Any, step: int = 0, epoch: int = 0) -> torch.Tensor:
        pred = predictions.get(self.prediction_key)
        target = getattr(batch, self.target_key, None)
        if pred is None:
            raise KeyError(f"loss term {self.name}: prediction '{self.prediction_key}' missing")
        if target is None:
            raise KeyError(f"loss term {self.name}: target '{self.target_key}' missing from the batch")
        if self.dtype is not None:
            pred, target = pred.to(self.dtype), target.to(self.dtype)
        return self.per_graph(pred, target.to(pred.dtype).reshape(pred.shape), batch).mean()

    def __add__(self, other: "BaseLossFunction | ComposedLossFunction") -> "ComposedLossFunction":
        return ComposedLossFunction([self]) + other

    def __mul__(self, factor: Any) -> "BaseLossFunction":
        import copy

        new = copy.copy(self)
        if callable(self.weight) or callable(factor):
            w0, f0 = self.weight, factor
            new.weight = lambda s, e: (w0(s, e) if callable(w0) else w0) * (f0(s, e) if callable(f0) else f0)
        else:
            new.weight = self.weight * factor
        return new

    __rmul__ = __mul__

    def to_spec(self) -> dict[str, Any]:
        w = self.weight.to_spec() if isinstance(self.weight, LossWeightSchedule) else self.weight
        return {"cls": type(self).__name__, "target_key": self.target_key, "prediction_key": self.prediction_key,
                "weight": w if not callable(w) else 1.0, "name": self.name}


def _huber(d: torch.Tensor, delta: float) -> torch.Tensor:
    a = d.abs()
    return torch.where(a <= delta, 0.5 * d * d, delta * (a - 0.5 * delta))


class EnergyMSELoss(BaseLossFunction):
    """Squared error of the per-atom-normalised energy."""

    def __init__(self, *a: Any, per_atom: bool = True, **k: Any) -> None:
        super().__init__(*a, **k)
        self.per_atom = per_atom

    def _norm(self, batch: Any, ref: torch.Tensor) -> torch.Tensor:
        return batch.num_nodes_per_graph.to(ref.dtype).clamp_min(1).reshape(-1, 1) if self.per_atom else 1.0

    def per_graph(self, pred, target, batch):
        return (((pred - target) / self._norm(batch, pred)) ** 2).reshape(pred.shape[0], -1).mean(-1)


class EnergyMAELoss(EnergyMSELoss):
    def per_graph(self, pred, target, batch):
        return ((pred - target) / self._norm(batch, pred)).abs().reshape(pred.shape[0], -1).mean(-1)


class EnergyHuberLoss(EnergyMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def per_graph(self, pred, target, batch):
        return _huber((pred - target) / self._norm(batch, pred), self.delta).reshape(pred.shape[0], -1).mean(-1)


class ForceMSELoss(BaseLossFunction):
    default_key = "forces"

    def per_graph(self, pred, target, batch):
        return per_graph_mean((pred - target) ** 2, batch.batch_idx, batch.num_graphs)


class ForceHuberLoss(ForceMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def per_graph(self, pred, target, batch):
        return per_graph_mean(_huber(pred - target, self.delta), batch.batch_idx, batch.num_graphs)


class ForceL2NormLoss(ForceMSELoss):
    def per_graph(self, pred, target, batch):
        return per_graph_mean((pred - target).norm(dim=-1, keepdim=True), batch.batch_idx, batch.num_graphs)


class StressMSELoss(BaseLossFunction):
    default_key = "stress"

    def per_graph(self, pred, target, batch):
        return frobenius_mse(pred, target)


class StressHuberLoss(StressMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def per_graph(self, pred, target, batch):
        return _huber(pred - target, self.delta).reshape(pred.shape[0], -1).mean(-1)


TERMS = {c.__name__: c for c in (EnergyMSELoss, EnergyMAELoss, EnergyHuberLoss, ForceMSELoss, ForceHuberLoss,
                                 ForceL2NormLoss, StressMSELoss, StressHuberLoss)}


class ComposedLossFunction:
    def __init__(self, terms: list[BaseLossFunction]) -> None:
        self.terms = list(terms)

    def __add__(self, other: "BaseLossFunction | ComposedLossFunction") -> "ComposedLossFunction":
        extra = other.terms if isinstance(other, ComposedLossFunction) else [other]
        return ComposedLossFunction(self.terms + list(extra))

    def __mul__(self, factor: Any) -> "ComposedLossFunction":
        return ComposedLossFunction([t * factor for t in self.terms])

    __rmul__ = __mul__

    def required_predictions(self) -> set[str]:
        return {t.prediction_key for t in self.terms}

    def __call__(self, predictions: dict, batch: Any, step: int = 0, epoch: int = 0) -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        total = None
        for t in self.terms:
            val = t(predictions, batch, step, epoch)
            out[t.name] = val.detach()
            w = t.weight_at(step, epoch)
            total = val * w if total is None else total + val * w
        out["total_loss"] = total
        return out

    def to_spec(self) -> list[dict[str, Any]]:
        return [t.to_spec() for t in self.terms]

    @classmethod
    def from_spec(cls, spec: list[dict[str, Any]]) -> "ComposedLossFunction":
        terms = []
        for s in spec:
            kw = {k: v for k, v in s.items() if k != "cls"}
            kw["weight"] = schedule_from_spec(kw.get("weight", 1.0))
            terms.append(TERMS[s["cls"]](**kw))
        return cls(terms)
