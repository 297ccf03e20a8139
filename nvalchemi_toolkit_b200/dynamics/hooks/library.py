# SPDX-License-Identifier: Apache-2.0
"""Stock dynamics hooks.

Constructor signatures and semantics follow the reference: ``NaNDetectorHook`` / ``MaxForceClampHook``
(``dynamics/hooks/safety.py:42-320``), ``EnergyDriftMonitorHook`` (``monitors.py:39-221``), ``FreezeAtomsHook``
(``freeze.py:36``), ``SnapshotHook`` / ``ConvergedSnapshotHook`` (``snapshot.py:40-223``), ``AlignCellHook``
(``cell_align.py:37``) and ``LoggingHook`` (``logging.py:72-415``: per-graph scalars, background writer thread, CSV or
TensorBoard backends).
"""
from __future__ import annotations

import csv
import queue
import threading
import warnings
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Literal

import torch

from nvalchemi_toolkit_b200._typing import AtomCategory
from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.dynamics._units import KB_EV
from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage


class NaNDetectorHook:
    """Raises ``RuntimeError`` naming the offending graphs when energy / forces (or ``extra_keys``) are non-finite."""

    def __init__(self, frequency: int = 1, extra_keys: list[str] | None = None,
                 stage: Enum = DynamicsStage.AFTER_COMPUTE) -> None:
        self.frequency, self.stage = frequency, stage
        self.keys = ["energy", "forces"] + list(extra_keys or [])

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        for key in self.keys:
            t = getattr(b, key, None)
            if t is None or not t.dtype.is_floating_point:
                continue
            bad = ~torch.isfinite(t.reshape(t.shape[0], -1)).all(dim=1)
            if bool(bad.any()):
                idx = torch.nonzero(bad).squeeze(1)
                graphs = b.batch_idx[idx].unique().tolist() if t.shape[0] == b.num_nodes and b.num_nodes != b.num_graphs \
                    else idx.tolist()
                raise RuntimeError(f"Non-finite values in '{key}' at step {ctx.step_count} for graphs {graphs}")


class MaxForceClampHook:
    """Rescales force vectors whose norm exceeds ``max_force`` (direction preserved)."""

    def __init__(self, max_force: float, stage: Enum = DynamicsStage.AFTER_COMPUTE, frequency: int = 1) -> None:
        if max_force <= 0:
            raise ValueError("max_force must be positive")
        self.max_force, self.stage, self.frequency = float(max_force), stage, frequency
        self.num_clamped = 0

    def __call__(self, ctx: Any, stage: Enum) -> None:
        f = ctx.batch.forces
        norm = f.norm(dim=-1, keepdim=True)
        scale = torch.clamp(self.max_force / norm.clamp_min(1e-30), max=1.0)
        f.mul_(scale)


class EnergyDriftMonitorHook:
    """Tracks total-energy drift per graph relative to the first observation."""

    def __init__(self, threshold: float, metric: Literal["absolute", "per_atom_per_step"] = "per_atom_per_step",
                 action: Literal["warn", "raise"] = "warn", frequency: int = 1, include_kinetic: bool = True,
                 stage: Enum = DynamicsStage.AFTER_STEP) -> None:
        self.threshold, self.metric, self.action = threshold, metric, action
        self.frequency, self.include_kinetic, self.stage = frequency, include_kinetic, stage
        self._e0: torch.Tensor | None = None
        self._step0 = 0
        self.last_drift: torch.Tensor | None = None

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        e = b.energy.reshape(-1).double().clone()
        if self.include_kinetic:
            e += _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, b.num_graphs).double()
        if self._e0 is None or self._e0.shape != e.shape:
            self._e0, self._step0 = e, ctx.step_count
            return
        drift = (e - self._e0).abs()
        if self.metric == "per_atom_per_step":
            steps = max(ctx.step_count - self._step0, 1)
            drift = drift / (b.num_nodes_per_graph.double().clamp_min(1) * steps)
        self.last_drift = drift
        if bool((drift > self.threshold).any()):
            msg = f"Energy drift {float(drift.max()):.3e} exceeds threshold {self.threshold:.3e} at step {ctx.step_count}"
            if self.action == "raise":
                raise RuntimeError(msg)
            warnings.warn(msg, RuntimeWarning, stacklevel=2)


class FreezeAtomsHook:
    """Pins atoms of one category: positions restored after the update, velocities (and optionally forces) zeroed."""

    def __init__(self, frequency: int = 1, freeze_category: int = AtomCategory.SPECIAL.value, zero_forces: bool = True,
                 stage: Enum = DynamicsStage.BEFORE_PRE_UPDATE) -> None:
        self.frequency, self.freeze_category, self.zero_forces, self.stage = frequency, freeze_category, zero_forces, stage
        self._saved: torch.Tensor | None = None

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in (DynamicsStage.BEFORE_PRE_UPDATE, DynamicsStage.AFTER_PRE_UPDATE, DynamicsStage.AFTER_COMPUTE,
                         DynamicsStage.AFTER_POST_UPDATE)

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        mask = b.atom_categories == self.freeze_category
        if stage == DynamicsStage.BEFORE_PRE_UPDATE:
            self._saved = b.positions[mask].clone()
            b.velocities[mask] = 0
            if self.zero_forces and b.forces is not None:
                b.forces[mask] = 0
        elif stage == DynamicsStage.AFTER_PRE_UPDATE:
            if self._saved is not None:
                b.positions[mask] = self._saved
            b.velocities[mask] = 0
        elif stage == DynamicsStage.AFTER_COMPUTE:
            if self.zero_forces:
                b.forces[mask] = 0
        else:
            b.velocities[mask] = 0


class SnapshotHook:
    """Writes the whole batch to a sink every ``frequency`` steps."""

    def __init__(self, sink: Any, frequency: int = 1, stage: Enum = DynamicsStage.AFTER_STEP) -> None:
        self.sink, self.frequency, self.stage = sink, frequency, stage

    def __call__(self, ctx: Any, stage: Enum) -> None:
        self.sink.write(ctx.batch)


class ConvergedSnapshotHook:
    """Writes only the systems that converged at this step (``ctx.converged_mask``)."""

    def __init__(self, sink: Any, frequency: int = 1, stage: Enum = DynamicsStage.ON_CONVERGE) -> None:
        self.sink, self.frequency, self.stage = sink, frequency, stage

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if ctx.converged_mask is not None and bool(ctx.converged_mask.any()):
            self.sink.write(ctx.batch, mask=ctx.converged_mask)


class AlignCellHook:
    """Keeps cells lower-triangular (needed by variable-cell integrators)."""

    def __init__(self, frequency: int = 1) -> None:
        self.frequency, self.stage = frequency, DynamicsStage.BEFORE_STEP

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        if getattr(b, "cell", None) is not None:
            _ops.align_cell(b.positions, b.cell, b.batch_idx)


class LoggingHook:
    """Per-graph scalars (energy, kinetic energy, temperature, fmax, + custom) to CSV / TensorBoard / a callable.

    Scalars are computed on the device and copied once per call; formatting and file IO happen on a worker thread."""

    def __init__(self, backend: str = "csv", frequency: int = 1, log_path: str | Path | None = None,
                 custom_scalars: dict[str, Callable[[Any], float | torch.Tensor]] | None = None,
                 writer_fn: Callable[[int, list[dict[str, float]]], None] | None = None,
                 stage: Enum = DynamicsStage.AFTER_STEP) -> None:
        self.backend, self.frequency, self.stage = backend, frequency, stage
        self.log_path = Path(log_path) if log_path is not None else None
        self.custom_scalars = dict(custom_scalars or {})
        self.writer_fn = writer_fn
        self.records: list[tuple[int, list[dict[str, float]]]] = []
        self._q: "queue.Queue | None" = None
        self._thread: threading.Thread | None = None
        self._tb = None
        self._csv_header_written = False

    def __enter__(self) -> "LoggingHook":
        self._q = queue.Queue()
        self._thread = threading.Thread(target=self._drain, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._q is not None:
            self._q.put(None)
            self._thread.join(timeout=30)
            self._q = self._thread = None
        if self._tb is not None:
            self._tb.flush()

    def _drain(self) -> None:
        while True:
            item = self._q.get()
            if item is None:
                return
            self._emit(*item)

    def _emit(self, step: int, rows: list[dict[str, float]]) -> None:
        if self.writer_fn is not None:
            self.writer_fn(step, rows)
        elif self.backend == "csv" and self.log_path is not None:
            new = not self._csv_header_written and not self.log_path.exists()
            with open(self.log_path, "a", newline="") as f:
                w = csv.DictWriter(f, fieldnames=["step", "graph"] + [k for k in rows[0] if k not in ("step", "graph")])
                if new:
                    w.writeheader()
                self._csv_header_written = True
                for g, r in enumerate(rows):
                    w.writerow({"step": step, "graph": g, **r})
        elif self.backend == "tensorboard" and self.log_path is not None:
            if self._tb is None:
                from torch.utils.tensorboard import SummaryWriter

                self._tb = SummaryWriter(str(self.log_path))
            for g, r in enumerate(rows):
                for k, v in r.items():
                    self._tb.add_scalar(f"graph{g}/{k}", v, step)
        else:
            self.records.append((step, rows))

    def __call__(self, ctx: Any, stage: Enum) -> None:
        b = ctx.batch
        m = b.num_graphs
        cols: dict[str, torch.Tensor] = {}
        if getattr(b, "energy", None) is not None:
            cols["energy"] = b.energy.reshape(-1)[:m].double()
        if getattr(b, "velocities", None) is not None:
            ke = _ops.compute_kinetic_energy(b.velocities, b.atomic_masses, b.batch_idx, m).double()
            cols["kinetic_energy"] = ke
            cols["temperature"] = 2.0 * ke / (3.0 * b.num_nodes_per_graph.double().clamp_min(1) * KB_EV)
        if getattr(b, "forces", None) is not None:
            cols["fmax"] = _ops.segmented_max(b.forces.norm(dim=-1).contiguous(), b.batch_idx, m).double()
        for name, fn in self.custom_scalars.items():
            v = fn(ctx)
            v = torch.as_tensor(v, dtype=torch.float64, device=b.device).reshape(-1)
            cols[name] = v.expand(m) if v.numel() == 1 else v
        table = torch.stack(list(cols.values()), dim=1).cpu().tolist()
        names = list(cols)
        rows = [dict(zip(names, row)) for row in table]
        if self._q is not None:
            self._q.put((ctx.step_count, rows))
        else:
            self._emit(ctx.step_count, rows)
