# SPDX-License-Identifier: Apache-2.0
"""Reporters: a Rich live dashboard, a TensorBoard writer and a JSON-lines file.

Reference: ``nvalchemi/hooks/reporting/_rich.py`` (live table + history plots, layouts for training and dynamics),
``_tensorboard.py`` (scalar writer with optional cross-rank reduction, rank-zero gating, injectable writer)."""
from __future__ import annotations

import json
from collections import deque
from enum import Enum
from pathlib import Path
from typing import Any, Mapping, Protocol, Sequence

from nvalchemi_toolkit_b200._optional import OptionalDependency
from nvalchemi_toolkit_b200.hooks.reporting._core import (ReportingState, ScalarCallback, ScalarSnapshot, collect_scalars,
                                                         reduce_scalars_across_ranks)
from nvalchemi_toolkit_b200.hooks.reporting._layouts import resolve_layout, text_plot

_BARS = " ▁▂▃▄▅▆▇█"


def sparkline(values: Sequence[float], width: int = 40) -> str:
    vals = [v for v in values if v == v][-width:]
    if not vals:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    return "".join(_BARS[1 + int((v - lo) / span * (len(_BARS) - 2))] for v in vals)


class RichLayout(str, Enum):
    AUTO = "auto"
    TRAIN = "train"
    DYNAMICS = "dynamics"
    COMPACT = "compact"


class _ScalarReporterBase:
    def __init__(self, custom_scalars: Mapping[str, ScalarCallback] | None, include_losses: bool,
                 include_optimizer_lrs: bool, include_dynamics_scalars: bool | None, rank_reduction: str | None,
                 rank_zero_only: bool) -> None:
        self.custom_scalars, self.include_losses = custom_scalars, include_losses
        self.include_optimizer_lrs, self.include_dynamics_scalars = include_optimizer_lrs, include_dynamics_scalars
        self.rank_reduction = None if rank_reduction is None else str(getattr(rank_reduction, "name", rank_reduction)).lower()
        if self.rank_reduction == "avg":
            self.rank_reduction = "mean"
        self.rank_zero_only = rank_zero_only
        self.requires_all_ranks = self.rank_reduction is not None  # a collective runs inside report()

    def snapshot(self, ctx: Any, stage: Enum, state: ReportingState) -> ScalarSnapshot:
        snap = collect_scalars(ctx, stage, state, include_losses=self.include_losses,
                               include_optimizer_lrs=self.include_optimizer_lrs,
                               include_dynamics_scalars=self.include_dynamics_scalars, custom_scalars=self.custom_scalars)
        if self.rank_reduction is not None:
            snap.scalars = reduce_scalars_across_ranks(snap.scalars, self.rank_reduction)
        return snap

    def _is_writer_rank(self) -> bool:
        import torch.distributed as dist

        return not self.rank_zero_only or not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


class RichReporter(_ScalarReporterBase):
    def __init__(self, *, custom_scalars: Mapping[str, ScalarCallback] | None = None, include_losses: bool = True,
                 include_optimizer_lrs: bool = True, include_dynamics_scalars: bool | None = None,
                 rank_reduction: str | None = None, title: str = "nvalchemi report", precision: int = 6,
                 max_scalars: int | None = None, history_size: int = 200, layout: RichLayout | str | None = None,
                 plot_keys: Sequence[str] | None = None, max_plots: int = 3, plot_height: int = 8,
                 refresh_per_second: float = 2.0, console: Any = None, screen: bool = False, transient: bool = False,
                 rank_zero_only: bool = True, strict_layout: bool = False) -> None:
        super().__init__(custom_scalars, include_losses, include_optimizer_lrs, include_dynamics_scalars, rank_reduction,
                         rank_zero_only)
        self.title, self.precision, self.max_scalars = title, precision, max_scalars
        # a name (RichLayout / str), None = auto, or any object with select_rows() / select_plots()
        self.layout = RichLayout(layout) if isinstance(layout, str) else (RichLayout.AUTO if layout is None else layout)
        if not isinstance(self.layout, RichLayout):
            resolve_layout(self.layout)  # fails now, not at the first report
        self.plot_keys, self.max_plots, self.plot_height = plot_keys, max_plots, plot_height
        self.refresh_per_second, self.console, self.screen, self.transient = refresh_per_second, console, screen, transient
        self.strict_layout = strict_layout
        self.history: dict[str, deque[float]] = {}
        self._history_size = history_size
        self._live: Any = None
        self.last_snapshot: ScalarSnapshot | None = None

    def _resolve_layout(self, snap: ScalarSnapshot) -> Any:
        return resolve_layout(self.layout, snap.scalars)

    def _select(self, snap: ScalarSnapshot, layout: Any) -> list[tuple[str, float]]:
        return layout.select_rows(snap.scalars, self.max_scalars, self.strict_layout)

    def _plot_panel(self, key: str, layout: Any, width: int) -> Any:
        from rich.panel import Panel

        h = list(self.history[key])
        log = bool(getattr(layout, "is_log", lambda *_: False)(key, h))
        rows = text_plot(h, width=width, height=self.plot_height, precision=4, log=log)
        title = f"{key}  last {h[-1]:.{self.precision}g}  min {min(h):.4g}  max {max(h):.4g}" + ("  (log)" if log else "")
        return Panel("\n".join(rows), title=title, height=self.plot_height + 2)

    def render(self, snap: ScalarSnapshot, state: ReportingState) -> Any:
        from rich.console import Group
        from rich.panel import Panel
        from rich.table import Table

        layout = self._resolve_layout(snap)
        head = f"{self.title} ({getattr(layout, 'name', 'custom')})  step {snap.step}"
        if snap.epoch is not None:
            head += f"  epoch {snap.epoch}"
        table = Table(title=head, caption=getattr(layout, "latest_title", None), expand=True)
        table.add_column("scalar")
        table.add_column("value", justify="right")
        table.add_column("history")
        for k, v in self._select(snap, layout):
            table.add_row(k, f"{v:.{self.precision}g}", sparkline(self.history.get(k, ()), 30))
        parts: list[Any] = [table]
        width = 80
        if self.console is not None and getattr(self.console, "width", None):
            width = max(20, int(self.console.width) - 20)
        for k in layout.select_plots(self.history, self.plot_keys, self.max_plots, self.strict_layout):
            parts.append(self._plot_panel(k, layout, width))
        recent = [m for m in list(state.messages)[-3:]]
        if recent:
            parts.append(Panel("\n".join(f"[{m.level}] {m.text}" for m in recent), title="messages"))
        return Group(*parts)

    def preview(self, layout: Any = None, n: int = 120) -> Any:
        """Static dashboard drawn from the layout's synthetic curves: what the live view will look like, without a run
        (documentation, choosing ``plot_keys`` / ``plot_height``).  The reporter's own history is left untouched."""
        chosen = resolve_layout(layout if layout is not None else (self.layout if self.layout != RichLayout.AUTO else "train"))
        curves = chosen.preview_history(n)
        keep_history, keep_layout = self.history, self.layout
        self.history = {k: deque(v, maxlen=max(self._history_size, n)) for k, v in curves.items()}
        self.layout = chosen
        try:
            snap = ScalarSnapshot(step=n - 1, epoch=getattr(chosen, "preview_epoch", None),
                                  stage=getattr(chosen, "preview_stage", "AFTER_STEP"),
                                  scalars={k: v[-1] for k, v in curves.items()})
            return self.render(snap, ReportingState())
        finally:
            self.history, self.layout = keep_history, keep_layout

    def __enter__(self) -> "RichReporter":
        if self._is_writer_rank():
            from rich.live import Live

            self._live = Live(console=self.console, refresh_per_second=self.refresh_per_second, screen=self.screen,
                              transient=self.transient)
            self._live.__enter__()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._live is not None:
            self._live.__exit__(*exc)
            self._live = None

    def report(self, ctx: Any, stage: Enum, state: ReportingState) -> None:
        snap = self.snapshot(ctx, stage, state)
        if not self._is_writer_rank():
            return
        for k, v in snap.scalars.items():
            self.history.setdefault(k, deque(maxlen=self._history_size)).append(v)
        self.last_snapshot = snap
        view = self.render(snap, state)
        if self._live is not None:
            self._live.update(view)
        else:
            from rich.console import Console

            (self.console or Console()).print(view)


class TensorBoardWriter(Protocol):
    """The part of ``torch.utils.tensorboard.SummaryWriter`` that :class:`TensorBoardReporter` calls: anything with these
    three methods can be injected as ``writer=`` (tests, other event sinks)."""

    def add_scalar(self, tag: str, scalar_value: float, global_step: int | None = None) -> None: ...

    def flush(self) -> None: ...

    def close(self) -> None: ...


class TensorBoardReporter(_ScalarReporterBase):
    def __init__(self, log_dir: str | Path, *, custom_scalars: Mapping[str, ScalarCallback] | None = None,
                 include_losses: bool = True, include_optimizer_lrs: bool = True, rank_reduction: str | None = None,
                 tag_prefix: str | None = None, flush: bool = True, rank_zero_only: bool = True, writer: Any = None) -> None:
        super().__init__(custom_scalars, include_losses, include_optimizer_lrs, None, rank_reduction, rank_zero_only)
        self.log_dir, self.tag_prefix, self.flush = Path(log_dir), tag_prefix, flush
        self._writer, self._owns_writer = writer, writer is None

    def _get_writer(self) -> Any:
        if self._writer is None:
            OptionalDependency.TENSORBOARD.import_module()
            from torch.utils.tensorboard import SummaryWriter

            self.log_dir.mkdir(parents=True, exist_ok=True)
            self._writer = SummaryWriter(log_dir=str(self.log_dir))
        return self._writer

    def report(self, ctx: Any, stage: Enum, state: ReportingState) -> None:
        snap = self.snapshot(ctx, stage, state)
        if not self._is_writer_rank():
            return
        w = self._get_writer()
        for k, v in snap.scalars.items():
            w.add_scalar(f"{self.tag_prefix}/{k}" if self.tag_prefix else k, v, global_step=snap.step)
        if self.flush and hasattr(w, "flush"):
            w.flush()

    def close(self) -> None:
        if self._writer is not None and self._owns_writer:
            self._writer.close()
            self._writer = None


class JSONLReporter(_ScalarReporterBase):
    """One JSON object per event; convenient for batch jobs without a terminal."""

    def __init__(self, path: str | Path, *, custom_scalars: Mapping[str, ScalarCallback] | None = None,
                 rank_reduction: str | None = None, rank_zero_only: bool = True) -> None:
        super().__init__(custom_scalars, True, True, None, rank_reduction, rank_zero_only)
        self.path = Path(path)
        self._fh: Any = None

    def report(self, ctx: Any, stage: Enum, state: ReportingState) -> None:
        snap = self.snapshot(ctx, stage, state)
        if not self._is_writer_rank():
            return
        if self._fh is None:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            self._fh = open(self.path, "a", encoding="utf-8")
        self._fh.write(json.dumps(snap.as_dict()) + "\n")
        self._fh.flush()

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
            self._fh = None
