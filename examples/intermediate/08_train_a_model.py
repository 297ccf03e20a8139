# SPDX-License-Identifier: Apache-2.0
"""Fit the demo network to energies and forces of a teacher: losses with a weight schedule, EMA, gradient clipping,
validation, a checkpoint and a restart."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper
from nvalchemi_toolkit_b200.training import (EnergyMSELoss, ForceMSELoss, LinearWeight, OptimizerConfig, TrainingStrategy,
                                             ValidationConfig)
from nvalchemi_toolkit_b200.training.hooks.library import EMAHook, GradientClipHook

torch.manual_seed(0)
teacher = DemoModelWrapper()


def labelled(n, seed):
    d = systems.argon_cluster(n, noise=0.2, seed=seed)
    out = teacher(Batch.from_data_list([d]))
    d.__dict__["energy"], d.__dict__["forces"] = out["energy"].detach().reshape(1, 1), out["forces"].detach()
    return d


train = [labelled(6 + i % 5, i) for i in range(32)]
val = [labelled(6 + i % 5, 100 + i) for i in range(8)]
loader = [Batch.from_data_list(train[i:i + 8]) for i in range(0, 32, 8)]
val_loader = [Batch.from_data_list(val)]
torch.manual_seed(1)
student = DemoModelWrapper()
loss = EnergyMSELoss(weight=1.0) + ForceMSELoss(weight=LinearWeight(1.0, 20.0, 40))   # forces matter more later on
strategy = TrainingStrategy(student, OptimizerConfig(kwargs={"lr": 3e-3}), loss_fn=loss, num_epochs=10, devices=["cpu"],
                            hooks=[GradientClipHook(max_norm=10.0), EMAHook(decay=0.99)],
                            validation_config=ValidationConfig(data=val_loader, every_n_epochs=5))
strategy.run(loader)
print("steps:", strategy.step_count, "| last training loss:", float(strategy.last_losses["total_loss"]))
print("validation:", {k: round(float(v), 6) for k, v in strategy.last_validation.items() if "loss" in k})
ckpt = Path(tempfile.mkdtemp()) / "ckpt"
strategy.save_checkpoint(ckpt)
resumed = TrainingStrategy(DemoModelWrapper(), OptimizerConfig(kwargs={"lr": 3e-3}), loss_fn=loss, num_epochs=12, devices=["cpu"])
resumed.load_checkpoint(ckpt)
resumed.run(loader)
print("resumed at step", 40, "and stopped at", resumed.step_count)
