# SPDX-License-Identifier: Apache-2.0
"""Reporting: orchestrator stage filter and error policies, scalar extraction, reporters, cross-rank reduction."""
import io
import json
import os

import pytest
import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage
from nvalchemi_toolkit_b200.hooks.core import DynamicsContext, TrainContext
from nvalchemi_toolkit_b200.hooks.reporting import (JSONLReporter, ReportingErrorPolicy, ReportingOrchestrator, RichReporter,
                                                    TensorBoardReporter, collect_scalars, reduce_scalars_across_ranks,
                                                    sparkline)
from tests.helpers import random_batch


class _Collect:
    def __init__(self):
        self.events, self.closed = [], False

    def report(self, ctx, stage, state):
        self.events.append((stage.name, state.num_events))

    def close(self):
        self.closed = True


class _Broken:
    def report(self, ctx, stage, state):
        raise RuntimeError("boom")


def _train_ctx(step=3):
    p = torch.nn.Parameter(torch.zeros(2))
    opt = torch.optim.SGD([p], lr=0.05)
    return TrainContext(batch=None, step_count=step, global_step_count=step, epoch=1, loss=torch.tensor(0.25),
                        losses={"energy": torch.tensor(0.2), "forces": torch.tensor([0.04, 0.06])}, optimizers=[opt])


def test_orchestrator_stage_filter_and_error_policies():
    good = _Collect()
    orch = ReportingOrchestrator([_Broken(), good], error_policy="disable")
    assert orch._runs_on_stage(DynamicsStage.AFTER_STEP) and not orch._runs_on_stage(DynamicsStage.BEFORE_STEP)
    ctx = DynamicsContext(batch=random_batch([3, 4]), step_count=2)
    with orch:
        orch(ctx, DynamicsStage.BEFORE_STEP)
        orch(ctx, DynamicsStage.AFTER_STEP)
        orch(ctx, DynamicsStage.AFTER_STEP)
    assert good.events == [("AFTER_STEP", 1), ("AFTER_STEP", 2)] and good.closed
    assert len(orch.state.messages) == 1 and "boom" in orch.state.messages[0].text  # disabled after the first failure
    with pytest.raises(RuntimeError):
        ReportingOrchestrator([_Broken()], error_policy=ReportingErrorPolicy.RAISE)(ctx, DynamicsStage.AFTER_STEP)
    warn = ReportingOrchestrator([_Broken()], error_policy="warn", stages={DynamicsStage.AFTER_STEP})
    warn(ctx, DynamicsStage.AFTER_STEP)
    warn(ctx, DynamicsStage.AFTER_STEP)
    assert len(warn.state.messages) == 2


def test_scalar_extraction_for_training_and_dynamics():
    snap = collect_scalars(_train_ctx(), None, custom_scalars={"custom/x": lambda c: 7})
    assert snap.step == 3 and snap.scalars["loss/total"] == 0.25 and abs(snap.scalars["loss/forces"] - 0.05) < 1e-7
    assert snap.scalars["lr/opt0"] == 0.05 and snap.scalars["custom/x"] == 7.0 and snap.scalars["progress/epoch"] == 1.0
    b = random_batch([3, 4])
    b["forces"] = torch.ones(7, 3)
    b["velocities"] = torch.ones(7, 3) * 0.1
    d = collect_scalars(DynamicsContext(batch=b, step_count=5, converged_mask=torch.tensor([True, False])), None)
    assert abs(d.scalars["dynamics/fmax"] - 3 ** 0.5) < 1e-6 and d.scalars["dynamics/active_fraction"] == 0.5
    assert d.scalars["dynamics/temperature"] > 0 and "loss/total" not in d.scalars


def test_rich_tensorboard_and_jsonl_reporters(tmp_path):
    from rich.console import Console

    buf = io.StringIO()
    rich = RichReporter(console=Console(file=buf, width=100, force_terminal=False), layout="train", plot_keys=["loss/total"])

    class _Writer:
        def __init__(self):
            self.rows = []

        def add_scalar(self, tag, value, global_step=None):
            self.rows.append((tag, value, global_step))

    w = _Writer()
    tb = TensorBoardReporter(tmp_path / "tb", writer=w, tag_prefix="run")
    js = JSONLReporter(tmp_path / "log.jsonl")
    from nvalchemi_toolkit_b200.training._stages import TrainingStage

    orch = ReportingOrchestrator([rich, tb, js])
    for step in (1, 2, 3):
        orch(_train_ctx(step), TrainingStage.AFTER_OPTIMIZER_STEP)
    orch.close()
    assert "loss/total" in buf.getvalue() and len(rich.history["loss/total"]) == 3
    assert ("run/loss/total", 0.25, 3) in w.rows
    rows = [json.loads(l) for l in (tmp_path / "log.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows] == [1, 2, 3] and rows[0]["lr/opt0"] == 0.05
    real = TensorBoardReporter(tmp_path / "tb_real")
    real.report(_train_ctx(1), TrainingStage.AFTER_OPTIMIZER_STEP, orch.state)
    real.close()
    assert any(p.name.startswith("events.out") for p in (tmp_path / "tb_real").iterdir())
    assert sparkline([1, 2, 3]) == "▁▄█"[0] + sparkline([1, 2, 3])[1:]  # monotone input gives a rising line
    assert len(sparkline(range(100), 10)) == 10


def _reduce_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = {"a": float(rank + 1), "only0": 5.0} if rank == 0 else {"a": float(rank + 1), "only1": 9.0}
        q.put((rank, reduce_scalars_across_ranks(mine, "mean"), reduce_scalars_across_ranks(mine, "max")))
    finally:
        dist.destroy_process_group()


def test_cross_rank_scalar_reduction_unions_keys():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reduce_worker, args=(r, 2, 29691, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r, (m, x)) for r, m, x in (q.get(timeout=120) for _ in range(2)))
    for p in procs:
        p.join(timeout=30)
    for r in range(2):
        mean, mx = res[r]
        assert mean == {"a": 1.5, "only0": 5.0, "only1": 9.0} and mx == {"a": 2.0, "only0": 5.0, "only1": 9.0}


def test_text_plot_rows_levels_and_log_scale():
    from nvalchemi_toolkit_b200.hooks.reporting import text_plot

    rows = text_plot([1, 2, 3, 4, 5, 4, 3, 2, 1], width=9, height=3)
    assert len(rows) == 3 and rows[0].startswith("5 ┤") and rows[-1].startswith("1 ┤")
    cells = [r.split("┤")[1] for r in rows]
    assert all(len(c) == 9 for c in cells)
    assert cells[0][4] == "█" and cells[0][0] == " " and cells[2][4] == "█"  # the peak fills all rows, the ends only the bottom
    assert text_plot([], height=4) == [] and text_plot([float("nan")], height=4) == []
    # more points than columns: resampled to the width, the newest point is kept
    long = text_plot(list(range(1000)), width=50, height=2)
    assert len(long[0].split("┤")[1]) == 50 and long[0].startswith("999")
    log = text_plot([1000.0, 100.0, 10.0, 1.0], width=4, height=3, log=True)
    heights = [sum(1 for r in log if r.split("┤")[1][i] != " ") for i in range(4)]
    assert heights == [3, 2, 1, 1] and log[0].startswith("1000") and log[-1].lstrip().startswith("1 ┤")


def test_dashboard_layouts_select_rows_plots_and_preview():
    from rich.console import Console

    from nvalchemi_toolkit_b200.hooks.reporting import (BaseDashboardLayout, DynamicsLayout, RichReporter, TrainingLayout,
                                                        resolve_layout)

    scalars = {"progress/step": 3.0, "lr/group0": 1e-3, "loss/forces": 0.2, "loss/total": 0.5, "custom/x": 1.0}
    t = TrainingLayout()
    assert [k for k, _ in t.select_rows(scalars)] == ["loss/total", "loss/forces", "lr/group0", "progress/step", "custom/x"]
    assert [k for k, _ in t.select_rows(scalars, strict=True)][-1] == "progress/step"
    assert [k for k, _ in t.select_rows(scalars, max_scalars=2)] == ["loss/total", "loss/forces"]
    hist = {"loss/total": [1.0, 0.5], "custom/x": [1.0, 2.0], "lr/group0": [1e-3], "progress/step": [0.0, 1.0]}
    assert t.select_plots(hist, None, 3) == ["loss/total", "custom/x"]  # one-point and progress series are not plotted
    assert t.select_plots(hist, ["custom/x", "missing"], 3) == ["custom/x"]
    assert isinstance(resolve_layout(None, scalars), TrainingLayout)
    assert isinstance(resolve_layout("auto", {"dynamics/fmax": 1.0}), DynamicsLayout)
    with pytest.raises(ValueError, match="unknown layout"):
        resolve_layout("fancy")
    with pytest.raises(TypeError, match="select_rows"):
        RichReporter(layout=object())

    class EnergyOnly(BaseDashboardLayout):
        name = "energy-only"
        row_prefixes = ("dynamics/energy",)
        preferred_plots = ("dynamics/energy",)

        def preview_history(self, n=120):
            return {"dynamics/energy": [float(-i) for i in range(n)], "dynamics/fmax": [1.0] * n}

    console = Console(width=90, record=True, force_terminal=False)
    rep = RichReporter(console=console, layout=EnergyOnly(), plot_height=4, strict_layout=True)
    rep.history["kept"] = [1.0]
    console.print(rep.preview())
    text = console.export_text()
    assert "energy-only" in text and "dynamics/energy" in text and "dynamics/fmax" not in text
    assert text.count("┤") == 4 and list(rep.history) == ["kept"]  # one plot of plot_height rows; own history untouched
    console.print(RichReporter(console=console, plot_height=3, max_plots=2).preview("train"))
    assert "loss/total" in console.export_text()
