# SPDX-License-Identifier: Apache-2.0
"""Dashboard layouts of the Rich reporter and the text plots they are made of.

Reference: ``nvalchemi/hooks/reporting/layouts/{base,train,dynamics}.py`` (a layout object decides which scalars form
the "latest" table, which are plotted, and can render a static preview from synthetic curves; plots there come from
``plotext``).  Here the plots are drawn by :func:`text_plot` (no dependency): a ``height``-row chart of Unicode block
eighths with the value range on the y axis, so a panel shows a trend with 8 * height levels instead of the 8 levels of
a one-line sparkline."""
from __future__ import annotations

import math
from typing import Any, Mapping, Protocol, Sequence

_EIGHTHS = " ▁▂▃▄▅▆▇█"


def _resample(values: Sequence[float], width: int) -> list[float]:
    """At most ``width`` points: the last value of each of ``width`` equal slices (keeps the most recent point)."""
    vals = [float(v) for v in values if v == v and math.isfinite(v)]
    if len(vals) <= width:
        return vals
    return [vals[min(len(vals) - 1, ((i + 1) * len(vals)) // width - 1)] for i in range(width)]


def text_plot(values: Sequence[float], width: int = 60, height: int = 8, precision: int = 4, log: bool = False) -> list[str]:
    """Column chart of ``values`` in ``height`` text rows (top row first).  Each column is filled from the bottom in
    eighths of a row; the first and last rows carry the maximum and minimum as labels.  ``log``: plot ``log10`` of the
    positive values (losses spanning decades)."""
    vals = _resample(values, max(int(width), 1))
    if log:
        vals = [math.log10(v) for v in vals if v > 0]
    if not vals or height < 1:
        return []
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    levels = [max(1, round((v - lo) / span * height * 8)) for v in vals]  # every point shows at least one eighth
    show = (lambda x: f"{10 ** x:.{precision}g}") if log else (lambda x: f"{x:.{precision}g}")
    labels = [""] * height
    labels[0], labels[-1] = show(hi), show(lo) if height > 1 else ""
    pad = max(len(s) for s in labels)
    rows = []
    for r in range(height):  # r = 0 is the top row
        base = (height - 1 - r) * 8
        cells = "".join(_EIGHTHS[min(8, max(0, lv - base))] for lv in levels)
        rows.append(f"{labels[r]:>{pad}} ┤{cells}")
    return rows


class DashboardLayout(Protocol):
    name: str
    include_dynamics_scalars: bool

    def select_rows(self, scalars: Mapping[str, float], max_scalars: int | None, strict: bool) -> list[tuple[str, float]]: ...

    def select_plots(self, history: Mapping[str, Sequence[float]], plot_keys: Sequence[str] | None, max_plots: int,
                     strict: bool = False) -> list[str]: ...

    def preview_history(self, n: int = 120) -> dict[str, list[float]]: ...


class BaseDashboardLayout:
    """Rows: scalars whose name starts with one of ``row_prefixes`` first (in that order, then by name), everything else
    after them unless ``strict``.  Plots: ``preferred_plots`` that have history, topped up with other keys unless ``strict``."""

    name = "base"
    include_dynamics_scalars = False
    row_prefixes: tuple[str, ...] = ()
    preferred_plots: tuple[str, ...] = ()
    log_plots: tuple[str, ...] = ()
    latest_title = "Latest"
    history_title = "History"

    def select_rows(self, scalars: Mapping[str, float], max_scalars: int | None = None, strict: bool = False) -> list[tuple[str, float]]:
        def rank(key: str) -> int:
            return next((i for i, p in enumerate(self.row_prefixes) if key.startswith(p)), len(self.row_prefixes))

        keys = sorted(scalars, key=lambda k: (rank(k), k))
        if strict:
            keys = [k for k in keys if rank(k) < len(self.row_prefixes)]
        rows = [(k, scalars[k]) for k in keys]
        return rows if max_scalars is None else rows[:max_scalars]

    def select_plots(self, history: Mapping[str, Sequence[float]], plot_keys: Sequence[str] | None = None, max_plots: int = 3,
                     strict: bool = False) -> list[str]:
        drawable = [k for k, h in history.items() if len(h) > 1]
        if plot_keys is not None:
            return [k for k in plot_keys if k in drawable][:max_plots]
        chosen = [k for k in self.preferred_plots if k in drawable]
        if not strict:
            chosen += [k for k in sorted(drawable) if k not in chosen and not k.startswith("progress/")]
        return chosen[:max_plots]

    def is_log(self, key: str, history: Sequence[float]) -> bool:
        return key in self.log_plots and min(history) > 0 and max(history) / min(history) > 100.0

    def preview_history(self, n: int = 120) -> dict[str, list[float]]:
        return {}

    preview_stage = "AFTER_STEP"
    preview_epoch: int | None = None


class TrainingLayout(BaseDashboardLayout):
    name = "train"
    row_prefixes = ("loss/total", "loss/", "validation/", "lr/", "progress/")
    preferred_plots = ("loss/total", "validation/total_loss", "lr/group0")
    log_plots = ("loss/total", "validation/total_loss")
    latest_title, history_title = "Losses and rates", "Curves"
    preview_stage, preview_epoch = "AFTER_OPTIMIZER_STEP", 3

    def preview_history(self, n: int = 120) -> dict[str, list[float]]:
        loss = [2.0 * math.exp(-i / 25.0) + 0.02 + 0.01 * math.sin(i * 0.9) for i in range(n)]
        return {"loss/total": loss, "loss/energy": [0.3 * v for v in loss], "loss/forces": [0.7 * v for v in loss],
                "validation/total_loss": [1.15 * v for v in loss[::10] for _ in range(10)][:n],
                "lr/group0": [1e-3 * 0.5 * (1 + math.cos(math.pi * i / n)) for i in range(n)],
                "progress/step": [float(i) for i in range(n)]}


class DynamicsLayout(BaseDashboardLayout):
    name = "dynamics"
    include_dynamics_scalars = True
    row_prefixes = ("dynamics/energy", "dynamics/fmax", "dynamics/temperature", "dynamics/", "progress/")
    preferred_plots = ("dynamics/energy", "dynamics/fmax", "dynamics/temperature", "dynamics/energy_drift",
                       "dynamics/converged_fraction", "dynamics/active_fraction")
    log_plots = ("dynamics/fmax",)
    latest_title, history_title = "State", "Traces"

    def preview_history(self, n: int = 120) -> dict[str, list[float]]:
        return {"dynamics/energy": [-3.0 - 1.2 * (1 - math.exp(-i / 30.0)) for i in range(n)],
                "dynamics/fmax": [1.5 * math.exp(-i / 18.0) + 0.01 for i in range(n)],
                "dynamics/temperature": [300.0 + 12.0 * math.sin(i / 7.0) * math.exp(-i / 80.0) for i in range(n)],
                "dynamics/converged_fraction": [min(1.0, max(0.0, (i - 40) / 60.0)) for i in range(n)],
                "progress/step": [float(i) for i in range(n)]}


class CompactLayout(BaseDashboardLayout):
    name = "compact"
    row_prefixes = ("loss/total", "dynamics/fmax", "progress/step")
    preferred_plots = ()

    def select_rows(self, scalars, max_scalars=None, strict=False):
        return super().select_rows(scalars, max_scalars, True)  # compact never lists the rest

    def select_plots(self, history, plot_keys=None, max_plots=3, strict=False):
        return super().select_plots(history, plot_keys, max_plots, strict) if plot_keys is not None else []


LAYOUTS: dict[str, type[BaseDashboardLayout]] = {"train": TrainingLayout, "dynamics": DynamicsLayout, "compact": CompactLayout}


def resolve_layout(layout: Any, scalars: Mapping[str, float] | None = None) -> BaseDashboardLayout:
    """A layout object, a name (``train`` / ``dynamics`` / ``compact``) or ``auto`` / ``None``: chosen from the scalars
    (training when any ``loss/`` scalar is present, else dynamics)."""
    name = getattr(layout, "value", layout)
    if name is None or name == "auto":
        has_loss = any(k.startswith("loss/") for k in (scalars or {}))
        return TrainingLayout() if has_loss else DynamicsLayout()
    if isinstance(name, str):
        if name not in LAYOUTS:
            raise ValueError(f"unknown layout {name!r}; choose from {sorted(LAYOUTS)} or pass a layout object")
        return LAYOUTS[name]()
    for attr in ("select_rows", "select_plots"):
        if not hasattr(layout, attr):
            raise TypeError(f"a layout object needs a {attr}() method")
    return layout
