# SPDX-License-Identifier: Apache-2.0
"""Reporting core: shared state, scalar extraction, cross-rank reduction, the orchestrator hook.

Reference: ``nvalchemi/hooks/reporting/_orchestrator.py:37-364``, ``_scalars.py:41-720``, ``_state.py:31-158``,
``_distributed.py``.  The orchestrator is an ordinary hook (it chooses its stages through ``_runs_on_stage``) that fans
a hook context out to reporters; reporters turn contexts into a :class:`ScalarSnapshot` with the extractors below.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Mapping, Protocol, Sequence, runtime_checkable

import torch

DEFAULT_REPORT_STAGES = frozenset({"AFTER_OPTIMIZER_STEP", "AFTER_STEP"})
ScalarCallback = Callable[[Any], float]


class ReportingErrorPolicy(str, Enum):
    RAISE = "raise"      # propagate the reporter's exception
    WARN = "warn"        # record a message, keep the reporter
    DISABLE = "disable"  # record a message, stop calling that reporter


@dataclass
class ReporterMessage:
    level: str
    text: str
    step: int | None = None
    stage: str | None = None
    source: str | None = None
    time: float = field(default_factory=time.time)


class ReportingState:
    """Event marks and a bounded message log shared by the reporters of one orchestrator."""

    def __init__(self, max_messages: int = 200) -> None:
        self.messages: deque[ReporterMessage] = deque(maxlen=max_messages)
        self.last_stage: str | None = None
        self.last_step: int | None = None
        self.num_events = 0
        self.started = time.time()
        self.last_event_time: float | None = None

    def mark_event(self, ctx: Any, stage: Enum) -> None:
        self.num_events += 1
        self.last_stage = getattr(stage, "name", str(stage))
        self.last_step = _step_of(ctx)
        self.last_event_time = time.time()

    def add_message(self, level: str, text: str, ctx: Any = None, stage: Enum | None = None, source: str | None = None
                    ) -> ReporterMessage:
        msg = ReporterMessage(level, text, _step_of(ctx) if ctx is not None else None,
                              getattr(stage, "name", None) if stage is not None else None, source)
        self.messages.append(msg)
        return msg


def _step_of(ctx: Any) -> int | None:
    for name in ("global_step_count", "step_count"):
        v = getattr(ctx, name, None)
        if isinstance(v, int) and v >= 0:
            if name == "global_step_count" and v == 0 and getattr(ctx, "step_count", 0):
                continue
            return v
    return None


@dataclass
class ScalarSnapshot:
    step: int | None
    stage: str | None
    scalars: dict[str, float]
    epoch: int | None = None
    wall_time: float = field(default_factory=time.time)

    def as_dict(self) -> dict[str, object]:
        return {"step": self.step, "stage": self.stage, "epoch": self.epoch, "wall_time": self.wall_time, **self.scalars}


def _to_float(value: Any, name: str) -> float:
    if isinstance(value, torch.Tensor):
        if value.numel() != 1:
            raise ValueError(f"scalar '{name}' has {value.numel()} elements")
        return float(value.detach())
    return float(value)


def extract_scalars(values: Mapping[str, object], *, prefix: str | None = None) -> dict[str, float]:
    """Flatten a nested mapping of scalar leaves (numbers, one-element tensors) into ``{"a/b/c": float}``; ``None``
    leaves are skipped (reference ``hooks/reporting/_scalars.py:447-485``).  A non-string key is a ``TypeError``, a
    tensor with several elements a ``ValueError``."""
    out: dict[str, float] = {}
    root = prefix.strip("/") if prefix else ""
    for name, value in values.items():
        if not isinstance(name, str):
            raise TypeError(f"scalar keys must be strings, got {type(name).__name__}")
        if value is None:
            continue
        key = f"{root}/{name.strip('/')}" if root else name.strip("/")
        if isinstance(value, Mapping):
            out.update(extract_scalars(value, prefix=key))
        else:
            out[key] = _to_float(value, key)
    return out


def _is_training(ctx: Any) -> bool:
    return hasattr(ctx, "optimizers") and hasattr(ctx, "epoch")


def extract_loss_scalars(ctx: Any) -> dict[str, float]:
    out: dict[str, float] = {}
    loss = getattr(ctx, "loss", None)
    if loss is not None:
        out["loss/total"] = _to_float(loss, "loss")
    for k, v in (getattr(ctx, "losses", None) or {}).items():
        if isinstance(v, torch.Tensor) and v.numel() != 1:
            v = v.detach().float().mean()
        out[f"loss/{k}"] = _to_float(v, k)
    val = getattr(ctx, "validation", None)
    if isinstance(val, Mapping):
        for k, v in val.items():
            try:
                out[f"validation/{k}"] = _to_float(v, k)
            except (TypeError, ValueError):
                continue
    return out


def extract_optimizer_lr_scalars(ctx: Any) -> dict[str, float]:
    out: dict[str, float] = {}
    for i, opt in enumerate(getattr(ctx, "optimizers", None) or []):
        groups = getattr(opt, "param_groups", [])
        for g, pg in enumerate(groups):
            key = f"lr/opt{i}" if len(groups) == 1 else f"lr/opt{i}/group{g}"
            out[key] = float(pg["lr"])
    return out


def extract_dynamics_scalars(ctx: Any) -> dict[str, float]:
    """Mean potential energy, max force, temperature, active fraction and per-status counts of a dynamics batch."""
    out: dict[str, float] = {}
    batch = getattr(ctx, "batch", None)
    if batch is None:
        return out
    energy = getattr(batch, "energy", None)
    if isinstance(energy, torch.Tensor) and energy.numel():
        out["dynamics/energy_mean"] = float(energy.detach().float().mean())
    forces = getattr(batch, "forces", None)
    if isinstance(forces, torch.Tensor) and forces.numel():
        out["dynamics/fmax"] = float(forces.detach().norm(dim=-1).max())
    vel, mass = getattr(batch, "velocities", None), getattr(batch, "atomic_masses", None)
    if isinstance(vel, torch.Tensor) and isinstance(mass, torch.Tensor) and vel.numel():
        from nvalchemi_toolkit_b200.dynamics._units import KB_EV

        ke = 0.5 * (mass.reshape(-1, 1) * vel.pow(2)).sum()
        out["dynamics/temperature"] = float(2.0 * ke / (3.0 * vel.shape[0] * KB_EV))
    status = getattr(batch, "status", None)
    if isinstance(status, torch.Tensor) and status.numel():
        flat = status.reshape(-1)
        for s in torch.unique(flat).tolist():
            out[f"dynamics/status_{int(s)}"] = float((flat == s).sum())
    mask = getattr(ctx, "converged_mask", None)
    if isinstance(mask, torch.Tensor) and mask.numel():
        out["dynamics/active_fraction"] = float(1.0 - mask.float().mean())
    return out


def extract_progress_scalars(ctx: Any, state: ReportingState | None = None) -> dict[str, float]:
    out: dict[str, float] = {}
    step = _step_of(ctx)
    if step is not None:
        out["progress/step"] = float(step)
    if _is_training(ctx):
        out["progress/epoch"] = float(getattr(ctx, "epoch", 0))
    wf = getattr(ctx, "workflow", None)
    target = getattr(wf, "num_steps", None) or getattr(wf, "n_steps", None)
    if isinstance(target, int) and target > 0 and step is not None:
        out["progress/fraction"] = min(1.0, step / target)
    if state is not None and step:
        elapsed = time.time() - state.started
        if elapsed > 0:
            out["progress/steps_per_s"] = step / elapsed
    return out


def collect_scalars(ctx: Any, stage: Enum | None = None, state: ReportingState | None = None, *,
                    include_losses: bool = True, include_optimizer_lrs: bool = True,
                    include_dynamics_scalars: bool | None = None, include_progress: bool = True,
                    custom_scalars: Mapping[str, ScalarCallback] | None = None) -> ScalarSnapshot:
    scalars: dict[str, float] = {}
    training = _is_training(ctx)
    if include_losses and training:
        scalars.update(extract_loss_scalars(ctx))
    if include_optimizer_lrs and training:
        scalars.update(extract_optimizer_lr_scalars(ctx))
    if include_dynamics_scalars or (include_dynamics_scalars is None and not training):
        scalars.update(extract_dynamics_scalars(ctx))
    if include_progress:
        scalars.update(extract_progress_scalars(ctx, state))
    for name, fn in (custom_scalars or {}).items():
        scalars[name] = _to_float(fn(ctx), name)
    return ScalarSnapshot(_step_of(ctx), getattr(stage, "name", None), scalars, getattr(ctx, "epoch", None))


def reduce_scalars_across_ranks(scalars: dict[str, float], op: str | None = "mean", group: Any = None,
                                device: torch.device | str | None = None) -> dict[str, float]:
    """Reduce a scalar dictionary over ranks: key sets are unioned (``all_gather_object``), values reduced as one tensor;
    a key missing on a rank contributes nothing (``mean`` divides by the number of contributing ranks)."""
    import torch.distributed as dist

    if op is None or not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(scalars)
    op = str(op).lower()
    if op not in ("mean", "sum", "max", "min"):
        raise ValueError("rank reduction must be one of mean, sum, max, min")
    keys_per_rank: list[Any] = [None] * dist.get_world_size(group)
    dist.all_gather_object(keys_per_rank, sorted(scalars), group=group)
    keys = sorted(set().union(*[set(k) for k in keys_per_rank]))
    if device is None:
        device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    fill = {"mean": 0.0, "sum": 0.0, "max": float("-inf"), "min": float("inf")}[op]
    vals = torch.tensor([scalars.get(k, fill) for k in keys], dtype=torch.float64, device=device)
    have = torch.tensor([1.0 if k in scalars else 0.0 for k in keys], dtype=torch.float64, device=device)
    dist.all_reduce(vals, op={"mean": dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX,
                              "min": dist.ReduceOp.MIN}[op], group=group)
    if op == "mean":
        dist.all_reduce(have, group=group)
        vals = vals / have.clamp_min(1.0)
    return {k: float(v) for k, v in zip(keys, vals.tolist())}


@runtime_checkable
class Reporter(Protocol):
    """``report(ctx, stage, state)``; optional ``rank_zero_only`` / ``requires_all_ranks`` flags and
    ``__enter__`` / ``__exit__`` / ``close`` for resources."""

    def report(self, ctx: Any, stage: Enum, state: ReportingState) -> None: ...


class ReportingOrchestrator:
    def __init__(self, reporters: Sequence[Reporter], *, frequency: int = 1, stages: set | None = None,
                 rank_zero_only: bool = False, error_policy: ReportingErrorPolicy | str = ReportingErrorPolicy.RAISE,
                 state: ReportingState | None = None) -> None:
        self.reporters = list(reporters)
        self.frequency = frequency
        self.stage: Enum | None = None
        self.rank_zero_only = rank_zero_only
        self.error_policy = ReportingErrorPolicy(error_policy)
        self.state = state if state is not None else ReportingState()
        self._stages = frozenset(stages if stages is not None else DEFAULT_REPORT_STAGES)
        self._depth = 0
        self._entered: list[Reporter] = []
        self._disabled: set[int] = set()
        self._closed = False

    @property
    def global_rank(self) -> int:
        import torch.distributed as dist

        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    @property
    def is_rank_zero(self) -> bool:
        return self.global_rank == 0

    def _runs_on_stage(self, stage: Enum) -> bool:
        return any(s is stage or (isinstance(s, str) and s == getattr(stage, "name", None)) for s in self._stages)

    def _skip(self, reporter: Reporter) -> bool:
        if getattr(reporter, "requires_all_ranks", False):
            return False
        gated = self.rank_zero_only or getattr(reporter, "rank_zero_only", False)
        return gated and not self.is_rank_zero

    def _fail(self, reporter: Reporter, exc: Exception, ctx: Any, stage: Enum | None, what: str) -> None:
        name = type(reporter).__name__
        if self.error_policy == ReportingErrorPolicy.RAISE:
            raise exc
        self.state.add_message("error", f"{name} failed during {what}: {exc!r}", ctx, stage, source=name)
        if self.error_policy == ReportingErrorPolicy.DISABLE:
            self._disabled.add(id(reporter))

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if self._closed or not self._runs_on_stage(stage):
            return
        self.state.mark_event(ctx, stage)
        for reporter in self.reporters:
            if id(reporter) in self._disabled or self._skip(reporter):
                continue
            try:
                reporter.report(ctx, stage, self.state)
            except Exception as exc:  # noqa: BLE001 - policy decides
                self._fail(reporter, exc, ctx, stage, "report")

    def __enter__(self) -> "ReportingOrchestrator":
        self._depth += 1
        if self._depth == 1:
            self._closed = False
            for reporter in self.reporters:
                if self._skip(reporter) or not hasattr(reporter, "__enter__"):
                    continue
                try:
                    reporter.__enter__()
                    self._entered.append(reporter)
                except Exception as exc:  # noqa: BLE001
                    self._fail(reporter, exc, None, None, "enter")
        return self

    def __exit__(self, *exc_info: Any) -> None:
        self._depth = max(0, self._depth - 1)
        if self._depth == 0:
            self._close(exc_info)

    def close(self) -> None:
        self._depth = 0
        self._close((None, None, None))

    def _close(self, exc_info: tuple) -> None:
        if self._closed:
            return
        self._closed = True
        first: Exception | None = None
        for reporter in reversed(self.reporters):
            try:
                if reporter in self._entered and hasattr(reporter, "__exit__"):
                    reporter.__exit__(*exc_info)
                elif hasattr(reporter, "close") and not self._skip(reporter):
                    reporter.close()
            except Exception as exc:  # noqa: BLE001
                self.state.add_message("error", f"{type(reporter).__name__} failed during close: {exc!r}")
                first = first or exc
        self._entered.clear()
        if first is not None and self.error_policy == ReportingErrorPolicy.RAISE:
            raise first
