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
