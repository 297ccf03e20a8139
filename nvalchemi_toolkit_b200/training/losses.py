# SPDX-License-Identifier: Apache-2.0
"""Loss terms, weight schedules and their composition.

Reference: ``nvalchemi/training/losses/{composition,terms,reductions,schedules}.py``.  A term compares
``predictions[prediction_key]`` with ``batch[target_key]``; terms compose with ``+`` and ``*`` into a
``ComposedLossFunction`` whose call returns ``{"total_loss": ..., "<name>": ...}``.  Weights may be constants or
schedules evaluated at ``(step, epoch)``.  Per-atom quantities are first reduced per graph (sum or mean over the graph's
atoms) so large systems do not dominate a batch.

Every term runs the same five steps (reference ``composition.py:280-527``): align dtypes (``dtype_policy``), validate
shapes, build a validity mask (padding rows of padded ``[B, V_max, ...]`` tensors; with ``ignore_nonfinite`` also every
target entry that is NaN / inf, i.e. a missing label), evaluate the elementwise residual with invalid targets replaced
(so neither the value nor the gradient sees them) and reduce: per graph first (``per_sample_loss`` keeps the detached
per-graph values of the last call), then over the graphs that have at least one valid entry."""
from __future__ import annotations

import math
from typing import Any, Callable, Protocol

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
DTYPE_POLICIES = ("strict", "prediction_to_target", "target_to_prediction")


def align_dtypes(pred: torch.Tensor, target: torch.Tensor, policy: str, who: str = "loss") -> tuple[torch.Tensor, torch.Tensor]:
    """``strict`` raises on a mismatch; the other two cast one side (reference ``composition.py:65-79``)."""
    if policy not in DTYPE_POLICIES:
        raise ValueError(f"dtype_policy must be one of {DTYPE_POLICIES}, got {policy!r}")
    if pred.dtype == target.dtype:
        return pred, target
    if policy == "strict":
        raise TypeError(f"{who}: prediction is {pred.dtype}, target is {target.dtype}; pick dtype_policy="
                        "'prediction_to_target' or 'target_to_prediction' to cast one side")
    return (pred.to(target.dtype), target) if policy == "prediction_to_target" else (pred, target.to(pred.dtype))


def assert_same_shape(pred: torch.Tensor, target: torch.Tensor, *, name: str, prediction_key: str | None = None,
                      target_key: str | None = None, strict: bool = False) -> None:
    """``ValueError`` when the two tensors cannot be compared: different dtypes first (usually the real bug), then the
    shapes: identical with ``strict``, else broadcast-compatible (reference ``composition.py:169-260``; elementwise
    terms should ask for ``strict``, because ``[B, 1]`` against ``[B, 3]`` broadcasts silently)."""
    who = f"loss term {name}" + (f" ({prediction_key} vs {target_key})" if prediction_key or target_key else "")
    if pred.dtype != target.dtype:
        raise ValueError(f"{who}: prediction is {pred.dtype}, target is {target.dtype}")
    if strict:
        if pred.shape != target.shape:
            raise ValueError(f"{who}: shapes {tuple(pred.shape)} and {tuple(target.shape)} differ")
        return
    try:
        torch.broadcast_shapes(pred.shape, target.shape)
    except RuntimeError as exc:
        raise ValueError(f"{who}: shapes {tuple(pred.shape)} and {tuple(target.shape)} do not broadcast") from exc


def node_counts(num_nodes_per_graph: torch.Tensor) -> torch.Tensor:
    """Per-graph atom counts from explicit counts ``[B]`` or a padded validity mask ``[B, V_max]``."""
    t = num_nodes_per_graph
    return t.sum(-1) if t.dtype == torch.bool or t.dim() == 2 else t


def padded_node_mask(num_nodes_per_graph: torch.Tensor, v_max: int) -> torch.Tensor:
    t = num_nodes_per_graph
    if t.dim() == 2:
        if t.shape[1] != v_max:
            raise ValueError(f"node mask has {t.shape[1]} columns, the padded tensor {v_max}")
        return t.to(torch.bool)
    return torch.arange(v_max, device=t.device)[None, :] < t.reshape(-1, 1)


class ReductionContext(dict):
    """What the reduction of a term needs to know about the batch besides the two tensors: ``num_graphs``, ``batch_idx``
    (dense node-level terms) and ``node_counts`` (per-graph atom counts, from explicit counts or a padding mask).
    Built once per call by :meth:`BaseLossFunction.reduction_context`; custom terms may add entries in ``normalize``."""

    @classmethod
    def from_batch(cls, batch: Any) -> "ReductionContext":
        ctx = cls(num_graphs=getattr(batch, "num_graphs", None), batch_idx=getattr(batch, "batch_idx", None))
        counts = getattr(batch, "num_nodes_per_graph", None)
        if counts is not None:
            ctx["node_counts"] = node_counts(counts)
        return ctx


class LossTargetAssemblyProtocol(Protocol):
    """A callable that collects the labels a loss needs from a batch (``assemble_loss_targets`` is the stock one; a
    strategy may be given another, e.g. one that reads labels from a side file keyed by sample id)."""

    def __call__(self, loss: Any, batch: Any, strict: bool = True) -> dict[str, torch.Tensor]: ...


class BaseLossFunction:
    """One weighted term.  Subclasses implement ``residual(pred, target, batch) -> elementwise tensor`` (same leading
    shape as ``pred``) and choose ``level`` (``"graph"``: one row per graph; ``"node"``: one row per atom, dense
    ``[V, ...]`` with ``batch.batch_idx`` or padded ``[B, V_max, ...]`` with ``batch.num_nodes_per_graph``)."""

    default_key = "energy"
    level = "graph"
    #: the prediction is a derivative of the model output (forces, stress): evaluation needs autograd switched on
    requires_eval_grad: bool | None = False

    def __init__(self, target_key: str | None = None, prediction_key: str | None = None, weight: Any = 1.0,
                 name: str | None = None, dtype: torch.dtype | None = None, ignore_nonfinite: bool = False,
                 dtype_policy: str = "target_to_prediction") -> None:
        if dtype_policy not in DTYPE_POLICIES:
            raise ValueError(f"dtype_policy must be one of {DTYPE_POLICIES}, got {dtype_policy!r}")
        self.target_key = target_key or self.default_key
        self.prediction_key = prediction_key or self.target_key
        self.weight = weight
        self.name = name or f"{type(self).__name__}[{self.prediction_key}]"
        self.dtype = dtype
        self.ignore_nonfinite = bool(ignore_nonfinite)
        self.dtype_policy = dtype_policy
        self.per_sample_loss: torch.Tensor | None = None

    def weight_at(self, step: int, epoch: int) -> float:
        return float(self.weight(step, epoch)) if callable(self.weight) else float(self.weight)

    def reduction_context(self, batch: Any) -> ReductionContext:
        return ReductionContext.from_batch(batch)

    # ---- the overridable steps
    def validate(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """Targets stored flat (``[B]`` energies, Voigt-free ``[B, 9]`` stresses) are viewed in the prediction's shape;
        a different element count is an error."""
        if target.shape != pred.shape:
            if target.numel() != pred.numel():
                raise ValueError(f"loss term {self.name}: prediction has shape {tuple(pred.shape)}, target {tuple(target.shape)}")
            target = target.reshape(pred.shape)
        return target

    def normalize(self, pred: torch.Tensor, target: torch.Tensor, batch: Any) -> tuple[torch.Tensor, torch.Tensor]:
        return pred, target

    def residual(self, pred: torch.Tensor, target: torch.Tensor, batch: Any) -> torch.Tensor:  # pragma: no cover
        raise NotImplementedError

    def graph_weights(self, batch: Any, ref: torch.Tensor) -> torch.Tensor | None:
        """Optional weights of the graphs in the final average (default: every graph with a valid entry counts once)."""
        return None

    # ---- shared machinery
    def _valid(self, pred: torch.Tensor, target: torch.Tensor, batch: Any) -> torch.Tensor | None:
        valid = None
        if self.level == "node" and pred.dim() >= 3:
            counts = getattr(batch, "num_nodes_per_graph", None)
            if counts is None:
                raise KeyError(f"loss term {self.name}: padded [B, V_max, ...] tensors need batch.num_nodes_per_graph")
            valid = padded_node_mask(counts, pred.shape[1]).reshape(pred.shape[:2] + (1,) * (pred.dim() - 2)).expand_as(pred)
        if self.ignore_nonfinite:
            finite = torch.isfinite(target)
            valid = finite if valid is None else valid & finite
        return valid

    def _reduce(self, res: torch.Tensor, valid: torch.Tensor | None, batch: Any) -> torch.Tensor:
        dense_nodes = self.level == "node" and res.dim() == 2
        ones = torch.ones_like(res) if valid is None else valid.to(res.dtype)
        if dense_nodes:
            idx, b = batch.batch_idx.long(), int(batch.num_graphs)
            tot = torch.zeros(b, dtype=res.dtype, device=res.device).index_add_(0, idx, res.sum(-1))
            cnt = torch.zeros(b, dtype=res.dtype, device=res.device).index_add_(0, idx, ones.sum(-1))
        else:
            tot, cnt = res.reshape(res.shape[0], -1).sum(-1), ones.reshape(res.shape[0], -1).sum(-1)
        per_graph = tot / cnt.clamp_min(1)
        self.per_sample_loss = per_graph.detach()
        if self.level == "node" and not getattr(self, "normalize_by_atom_count", True):
            return tot.sum() / cnt.sum().clamp_min(1)  # one mean over every valid component of the batch
        w = (cnt > 0).to(res.dtype)
        gw = self.graph_weights(batch, res)
        if gw is not None:
            w = w * gw.reshape(-1).to(res.dtype)
        return (per_graph * w).sum() / w.sum().clamp_min(torch.finfo(res.dtype).tiny)

    def __call__(self, predictions: dict, batch: Any, step: int = 0, epoch: int = 0) -> torch.Tensor:
        pred = predictions.get(self.prediction_key)
        target = getattr(batch, self.target_key, None)
        if pred is None:
            raise KeyError(f"loss term {self.name}: prediction '{self.prediction_key}' missing")
        if target is None:
            raise KeyError(f"loss term {self.name}: target '{self.target_key}' missing from the batch")
        if self.dtype is not None:
            pred, target = pred.to(self.dtype), target.to(self.dtype)
        pred, target = align_dtypes(pred, target, self.dtype_policy, f"loss term {self.name}")
        target = self.validate(pred, target)
        valid = self._valid(pred, target, batch)
        if valid is not None:
            target = torch.where(valid, target, pred.detach())  # an invalid entry has residual 0 and gradient 0
        pred, target = self.normalize(pred, target, batch)
        res = self.residual(pred, target, batch)
        if valid is not None:
            if valid.shape != res.shape:  # a per-row residual (vector norm) is valid when all its components are
                valid = valid.all(-1, keepdim=True)
            res = res * valid.to(res.dtype)
        return self._reduce(res, valid, batch)

    def __add__(self, other: "BaseLossFunction | ComposedLossFunction") -> "ComposedLossFunction":
        return ComposedLossFunction([self]) + other

    def __radd__(self, other: Any) -> "ComposedLossFunction | BaseLossFunction":
        return self if other == 0 else ComposedLossFunction([self]).__add__(other)  # sum([...]) starts from 0

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

    def _options(self) -> dict[str, Any]:
        return {}

    def to_spec(self) -> dict[str, Any]:
        w = self.weight.to_spec() if isinstance(self.weight, LossWeightSchedule) else self.weight
        spec = {"cls": type(self).__name__, "target_key": self.target_key, "prediction_key": self.prediction_key,
                "weight": w if not callable(w) else 1.0, "name": self.name, **self._options()}
        if self.ignore_nonfinite:
            spec["ignore_nonfinite"] = True
        if self.dtype_policy != "target_to_prediction":
            spec["dtype_policy"] = self.dtype_policy
        return spec


def _huber(d: torch.Tensor, delta: float) -> torch.Tensor:
    a = d.abs()
    return torch.where(a <= delta, 0.5 * d * d, delta * (a - 0.5 * delta))


class EnergyMSELoss(BaseLossFunction):
    """Squared error of the energy, per atom by default.  ``atom_weighted`` (needs ``per_atom``): graphs enter the batch
    average in proportion to their atom counts, ``sum_i N_i (dE_i / N_i)^2 / sum_i N_i`` (the reduction of reference
    ``terms.py:143-268``); default: every labelled graph counts once."""

    def __init__(self, *a: Any, per_atom: bool = True, atom_weighted: bool = False, **k: Any) -> None:
        super().__init__(*a, **k)
        if atom_weighted and not per_atom:
            raise ValueError("atom_weighted=True needs per_atom=True")
        self.per_atom, self.atom_weighted = per_atom, atom_weighted

    def _counts(self, batch: Any, ref: torch.Tensor) -> torch.Tensor:
        ctx = self.reduction_context(batch)
        if "node_counts" not in ctx:
            raise KeyError(f"loss term {self.name}: per-atom normalisation needs batch.num_nodes_per_graph")
        return ctx["node_counts"].to(ref.dtype).clamp_min(1)

    def normalize(self, pred, target, batch):
        if not self.per_atom:
            return pred, target
        n = self._counts(batch, pred).reshape((-1,) + (1,) * (pred.dim() - 1))
        return pred / n, target / n

    def graph_weights(self, batch, ref):
        return self._counts(batch, ref) if self.atom_weighted else None

    def residual(self, pred, target, batch):
        return (pred - target) ** 2

    def _options(self):
        return {"per_atom": self.per_atom, **({"atom_weighted": True} if self.atom_weighted else {})}


class EnergyMAELoss(EnergyMSELoss):
    def residual(self, pred, target, batch):
        return (pred - target).abs()


class EnergyHuberLoss(EnergyMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def residual(self, pred, target, batch):
        return _huber(pred - target, self.delta)

    def _options(self):
        return {**super()._options(), "delta": self.delta}


class ForceMSELoss(BaseLossFunction):
    """Squared error of the force components.  Dense ``[V, 3]`` forces are grouped by ``batch.batch_idx``; padded
    ``[B, V_max, 3]`` forces skip the padding rows named by ``batch.num_nodes_per_graph`` (counts ``[B]`` or a mask
    ``[B, V_max]``).  ``normalize_by_atom_count=True``: mean per graph, then mean over graphs (graph-balanced);
    ``False``: one mean over every valid component of the batch (reference ``terms.py:475-695``)."""

    default_key = "forces"
    level = "node"
    requires_eval_grad = True

    def __init__(self, *a: Any, normalize_by_atom_count: bool = True, **k: Any) -> None:
        super().__init__(*a, **k)
        self.normalize_by_atom_count = bool(normalize_by_atom_count)

    def residual(self, pred, target, batch):
        return (pred - target) ** 2

    def _options(self):
        return {} if self.normalize_by_atom_count else {"normalize_by_atom_count": False}


class ForceHuberLoss(ForceMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def residual(self, pred, target, batch):
        return _huber(pred - target, self.delta)

    def _options(self):
        return {**super()._options(), "delta": self.delta}


class ForceL2NormLoss(ForceMSELoss):
    """Mean length of the force error vector (not squared): less sensitive to a few atoms with large forces."""

    def residual(self, pred, target, batch):
        return (pred - target).norm(dim=-1, keepdim=True)


class StressMSELoss(BaseLossFunction):
    default_key = "stress"
    requires_eval_grad = True

    def residual(self, pred, target, batch):
        return (pred - target) ** 2


class StressHuberLoss(StressMSELoss):
    def __init__(self, *a: Any, delta: float = 0.01, **k: Any) -> None:
        super().__init__(*a, **k)
        self.delta = delta

    def residual(self, pred, target, batch):
        return _huber(pred - target, self.delta)

    def _options(self):
        return {"delta": self.delta}


TERMS = {c.__name__: c for c in (EnergyMSELoss, EnergyMAELoss, EnergyHuberLoss, ForceMSELoss, ForceHuberLoss,
                                 ForceL2NormLoss, StressMSELoss, StressHuberLoss)}


class ComposedLossFunction:
    """Weighted sum of terms.  The call returns ``{"total_loss": ..., "<term name>": detached value, ...}``.

    ``normalize_weights=True`` divides the weights in force at ``(step, epoch)`` by their sum, so schedules steer the
    RELATIVE share of the terms and the learning rate alone sets the scale (the reference's default,
    ``composition.py:609-660``; here it is opt-in).  ``dtype_policy`` overrides the policy of every term for calls made
    through this composition, without touching the term objects (they may be shared)."""

    def __init__(self, terms: list[BaseLossFunction], normalize_weights: bool = False, dtype_policy: str | None = None) -> None:
        flat: list[BaseLossFunction] = []
        for t in terms:
            if isinstance(t, ComposedLossFunction):
                flat.extend(t.terms)
            elif isinstance(t, BaseLossFunction):
                flat.append(t)
            else:
                raise TypeError(f"loss terms must be BaseLossFunction or ComposedLossFunction, got {type(t).__name__}")
        if not flat:
            raise ValueError("a composed loss needs at least one term")
        names = [t.name for t in flat]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"loss term names must be unique (they key the output dictionary): {dup}; pass name=...")
        if dtype_policy is not None and dtype_policy not in DTYPE_POLICIES:
            raise ValueError(f"dtype_policy must be one of {DTYPE_POLICIES} or None, got {dtype_policy!r}")
        self.terms = flat
        self.normalize_weights = bool(normalize_weights)
        self.dtype_policy = dtype_policy

    def __add__(self, other: "BaseLossFunction | ComposedLossFunction") -> "ComposedLossFunction":
        extra = other.terms if isinstance(other, ComposedLossFunction) else [other]
        return ComposedLossFunction(self.terms + list(extra), self.normalize_weights, self.dtype_policy)

    def __radd__(self, other: Any) -> "ComposedLossFunction":
        return self if other == 0 else self.__add__(other)

    def __mul__(self, factor: Any) -> "ComposedLossFunction":
        return ComposedLossFunction([t * factor for t in self.terms], self.normalize_weights, self.dtype_policy)

    __rmul__ = __mul__

    def required_predictions(self) -> set[str]:
        return {t.prediction_key for t in self.terms}

    @property
    def requires_eval_grad(self) -> bool:
        """Some term compares a derivative of the model output: evaluation must keep autograd on."""
        return any(bool(t.requires_eval_grad) for t in self.terms)

    def weights_at(self, step: int = 0, epoch: int = 0) -> dict[str, float]:
        w = {t.name: t.weight_at(step, epoch) for t in self.terms}
        if self.normalize_weights:
            total = sum(w.values())
            if total == 0.0:
                raise ValueError(f"loss weights sum to zero at step {step}, epoch {epoch}: {w}")
            w = {k: v / total for k, v in w.items()}
        return w

    def __call__(self, predictions: dict, batch: Any, step: int = 0, epoch: int = 0) -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        total = None
        weights = self.weights_at(step, epoch)
        for t in self.terms:
            if self.dtype_policy is not None and t.dtype_policy != self.dtype_policy:
                keep, t.dtype_policy = t.dtype_policy, self.dtype_policy
                try:
                    val = t(predictions, batch, step, epoch)
                finally:
                    t.dtype_policy = keep
            else:
                val = t(predictions, batch, step, epoch)
            out[t.name] = val.detach()
            w = weights[t.name]
            total = val * w if total is None else total + val * w
        out["total_loss"] = total
        return out

    def per_sample_losses(self) -> dict[str, torch.Tensor]:
        """Detached per-graph values of the last call, by term (for error histograms and outlier reports)."""
        return {t.name: t.per_sample_loss for t in self.terms if t.per_sample_loss is not None}

    def to_spec(self) -> list[dict[str, Any]]:
        return [t.to_spec() for t in self.terms]

    @classmethod
    def from_spec(cls, spec: list[dict[str, Any]], **kwargs: Any) -> "ComposedLossFunction":
        terms = []
        for s in spec:
            kw = {k: v for k, v in s.items() if k != "cls"}
            kw["weight"] = schedule_from_spec(kw.get("weight", 1.0))
            terms.append(TERMS[s["cls"]](**kw))
        return cls(terms, **kwargs)


DTypePolicy = str  # one of ``DTYPE_POLICIES``
ComposedLossOutput = dict  # ``{"total_loss": tensor, "<term name>": detached tensor, ...}``


def loss_component_to_spec(term: "BaseLossFunction") -> dict[str, Any]:
    """The JSON record of one term (what ``ComposedLossFunction.to_spec`` lists; ``from_spec`` rebuilds it)."""
    return term.to_spec()


def as_composed_loss(loss: "BaseLossFunction | ComposedLossFunction | list") -> ComposedLossFunction:
    """A single term, a list of terms / spec dictionaries or a composition -> a composition."""
    if isinstance(loss, ComposedLossFunction):
        return loss
    if isinstance(loss, BaseLossFunction):
        return ComposedLossFunction([loss])
    if isinstance(loss, (list, tuple)):
        if loss and all(isinstance(x, dict) for x in loss):
            return ComposedLossFunction.from_spec(list(loss))
        return ComposedLossFunction(list(loss))
    raise TypeError(f"cannot build a loss from {type(loss).__name__}")


def loss_target_keys(loss: "BaseLossFunction | ComposedLossFunction") -> tuple[str, ...]:
    """Batch attributes the loss reads as labels, in term order without repeats."""
    seen: dict[str, None] = {}
    for t in as_composed_loss(loss).terms:
        seen.setdefault(t.target_key)
    return tuple(seen)


def assemble_loss_targets(loss: "BaseLossFunction | ComposedLossFunction", batch: Any, strict: bool = True) -> dict[str, torch.Tensor]:
    """The labels of ``batch`` the loss needs (reference ``composition.py:1113-1173``).  ``strict``: a missing label
    raises with the list of what the batch does carry; otherwise it is left out (pair with ``ignore_nonfinite`` terms
    only when the collate step fills missing labels with NaN)."""
    out: dict[str, torch.Tensor] = {}
    for key in loss_target_keys(loss):
        value = getattr(batch, key, None)
        if value is None:
            if strict:
                have = sorted(k for k in getattr(batch, "keys", lambda: [])())
                raise KeyError(f"batch carries no label '{key}' (fields: {have})")
            continue
        out[key] = value
    return out


def compute_supervised_loss(model_fn: Callable[[Any], dict], loss: "BaseLossFunction | ComposedLossFunction", batch: Any,
                            step: int = 0, epoch: int = 0) -> tuple[dict[str, torch.Tensor], dict]:
    """One supervised evaluation: check the labels, run the model, check that it produced what the terms compare,
    evaluate.  Returns ``(losses, predictions)``."""
    composed = as_composed_loss(loss)
    assemble_loss_targets(composed, batch)
    preds = model_fn(batch)
    missing = sorted(composed.required_predictions() - set(preds))
    if missing:
        raise KeyError(f"the model returned {sorted(preds)}, the loss also needs {missing}")
    return composed(preds, batch, step=step, epoch=epoch), preds
