# SPDX-License-Identifier: Apache-2.0
"""Train a small MACE on energies and forces of a Lennard-Jones teacher (energy MSE + 100 x force MSE, Adam), validate,
checkpoint asynchronously and keep training while the files are written.

Training differentiates the forces with respect to the weights, so the wrapper runs its PyTorch path in ``train()`` mode;
the same weights serve the native inference kernels after ``eval()``."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
from nvalchemi_toolkit_b200.models.mace import MACEWrapper
from nvalchemi_toolkit_b200.neighbors import compute_neighbors
from nvalchemi_toolkit_b200.training import EnergyMSELoss, ForceMSELoss, OptimizerConfig, TrainingStrategy, ValidationConfig
from nvalchemi_toolkit_b200.training.hooks.library import CheckpointHook, GradientClipHook

torch.manual_seed(0)
teacher = LennardJonesModelWrapper(epsilon=0.4, sigma=2.34, cutoff=6.0)


def labelled(seed: int):
    d = systems.fcc(2, a=3.61, z=29, noise=0.15, seed=seed)
    b = Batch.from_data_list([d])
    compute_neighbors(b, config=teacher.model_config.neighbor_config)
    out = teacher(b)
    d.__dict__["energy"], d.__dict__["forces"] = out["energy"].detach().reshape(1, 1), out["forces"].detach()
    return d


student = MACEWrapper(atomic_numbers=[29], channels=8, r_max=5.0, avg_num_neighbors=40.0)


def batches(items, size):
    out = []
    for i in range(0, len(items), size):
        b = Batch.from_data_list(items[i:i + size])
        compute_neighbors(b, config=student.model_config.neighbor_config)   # the student's own 5 A list, built once
        out.append(b)
    return out


loader = batches([labelled(s) for s in range(16)], 4)
val_loader = batches([labelled(100 + s) for s in range(4)], 4)
out_dir = Path(tempfile.mkdtemp()) / "ckpt"
strategy = TrainingStrategy(student, OptimizerConfig(kwargs={"lr": 1e-2}), loss_fn=EnergyMSELoss(weight=1.0) + ForceMSELoss(weight=100.0),
                            num_epochs=3, devices=["cpu"],
                            hooks=[GradientClipHook(max_norm=100.0), CheckpointHook(out_dir, every_n_epochs=1, asynchronous=True)],
                            validation_config=ValidationConfig(data=val_loader, every_n_epochs=1))
strategy.run(loader)
print("steps:", strategy.step_count, "| last training loss:", round(float(strategy.last_losses["total_loss"]), 4))
print("validation:", {k: round(float(v), 4) for k, v in strategy.last_validation.items() if "loss" in k})
print("checkpoints written:", sorted(p.name for p in (out_dir / "models" / "main" / "checkpoints").glob("*.pt")))
