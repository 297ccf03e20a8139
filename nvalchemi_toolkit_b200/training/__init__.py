# SPDX-License-Identifier: Apache-2.0
"""Training: hook-driven strategy, losses, optimiser configs, validation, checkpoints, fine-tuning, CLI."""
from nvalchemi_toolkit_b200.training._stages import TrainingStage
from nvalchemi_toolkit_b200.training.losses import (
    BaseLossFunction, ComposedLossFunction, ConstantWeight, CosineWeight, EnergyHuberLoss, EnergyMAELoss, EnergyMSELoss,
    ForceHuberLoss, ForceL2NormLoss, ForceMSELoss, LinearWeight, PiecewiseWeight, StressHuberLoss, StressMSELoss,
    as_composed_loss, assemble_loss_targets, compute_supervised_loss, loss_target_keys,
)
from nvalchemi_toolkit_b200.training.optimizers import OptimizerConfig
from nvalchemi_toolkit_b200.training.strategy import TrainingStrategy, default_training_fn
from nvalchemi_toolkit_b200.training.validation import ValidationConfig, ValidationLoop

__all__ = ["TrainingStage", "TrainingStrategy", "default_training_fn", "OptimizerConfig", "ValidationConfig",
           "ValidationLoop", "BaseLossFunction", "ComposedLossFunction", "EnergyMSELoss", "EnergyMAELoss",
           "EnergyHuberLoss", "ForceMSELoss", "ForceHuberLoss", "ForceL2NormLoss", "StressMSELoss", "StressHuberLoss",
           "ConstantWeight", "LinearWeight", "CosineWeight", "PiecewiseWeight", "as_composed_loss", "assemble_loss_targets",
           "compute_supervised_loss", "loss_target_keys"]
