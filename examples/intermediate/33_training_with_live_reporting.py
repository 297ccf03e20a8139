# SPDX-License-Identifier: Apache-2.0
"""Training with the reporting stack: a live Rich table (losses, learning rate, progress, history sparkline), a JSONL
metrics file and TensorBoard event files, all fed by one ``ReportingOrchestrator`` registered as a training hook.
Reporters only see scalars the orchestrator extracted once per event; a reporter that fails is disabled, not fatal
(``error_policy="disable"``)."""
import json
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.hooks.reporting import JSONLReporter, ReportingOrchestrator, RichReporter, TensorBoardReporter
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper
from nvalchemi_toolkit_b200.training import EnergyMSELoss, ForceMSELoss, OptimizerConfig, TrainingStrategy

torch.manual_seed(0)
teacher = DemoModelWrapper()


def labelled(n, seed):
    d = systems.argon_cluster(n, noise=0.2, seed=seed)
    out = teacher(Batch.from_data_list([d]))
    d.__dict__["energy"], d.__dict__["forces"] = out["energy"].detach().reshape(1, 1), out["forces"].detach()
    return d


data = [labelled(6 + i % 5, i) for i in range(32)]
loader = [Batch.from_data_list(data[i:i + 8]) for i in range(0, 32, 8)]
out = Path(tempfile.mkdtemp())
report = ReportingOrchestrator(
    [RichReporter(layout="train", title="demo network", plot_keys=["loss/total"]),
     JSONLReporter(out / "metrics.jsonl"), TensorBoardReporter(out / "tb")],
    frequency=4, error_policy="disable",
    )
torch.manual_seed(1)
strategy = TrainingStrategy(DemoModelWrapper(), OptimizerConfig(kwargs={"lr": 3e-3}), loss_fn=EnergyMSELoss() + ForceMSELoss(weight=10.0),
                            num_epochs=6, devices=["cpu"], hooks=[report])
with report:
    strategy.run(loader)
rows = [json.loads(line) for line in (out / "metrics.jsonl").read_text().splitlines()]
print(f"{len(rows)} metric rows; loss {rows[0]['loss/total']:.4f} -> {rows[-1]['loss/total']:.4f}; "
      f"keys: {sorted(k for k in rows[-1] if k != 'step')[:6]} ...")
print("tensorboard files:", sorted(p.name for p in (out / "tb").iterdir())[:2])
