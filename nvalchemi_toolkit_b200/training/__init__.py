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

from nvalchemi_toolkit_b200.training._spec import (BaseSpec, create_model_spec, create_model_spec_from_json,
                                                   register_type_serializer)
from nvalchemi_toolkit_b200.training.checkpoint import (CheckpointManifest, CheckpointValidator, load_checkpoint,
                                                        same_class_validator, save_checkpoint)
from nvalchemi_toolkit_b200.training.losses import (ComposedLossOutput, DTypePolicy, LossTargetAssemblyProtocol,
                                                    LossWeightSchedule, ReductionContext, loss_component_to_spec)
from nvalchemi_toolkit_b200.training.optimizers import (setup_optimizers, step_lr_schedulers, step_optimizers,
                                                        zero_gradients)
from nvalchemi_toolkit_b200.training.runtime import (configure_dataloader, configure_parallelism, freeze_unconfigured_models,
                                                     move_to_devices, train_configured_models)
from nvalchemi_toolkit_b200.training.validation import BatchValidationCallback

__all__ = ["TrainingStage", "TrainingStrategy", "default_training_fn", "OptimizerConfig", "ValidationConfig",
           "ValidationLoop", "BaseLossFunction", "ComposedLossFunction", "EnergyMSELoss", "EnergyMAELoss",
           "EnergyHuberLoss", "ForceMSELoss", "ForceHuberLoss", "ForceL2NormLoss", "StressMSELoss", "StressHuberLoss",
           "ConstantWeight", "LinearWeight", "CosineWeight", "PiecewiseWeight", "as_composed_loss", "assemble_loss_targets",
           "compute_supervised_loss", "loss_target_keys", "BaseSpec", "create_model_spec", "create_model_spec_from_json",
           "register_type_serializer", "CheckpointManifest", "CheckpointValidator", "load_checkpoint", "save_checkpoint",
           "same_class_validator", "ComposedLossOutput", "DTypePolicy", "LossWeightSchedule", "LossTargetAssemblyProtocol", "ReductionContext", "loss_component_to_spec",
           "setup_optimizers", "step_lr_schedulers", "step_optimizers", "zero_gradients", "configure_dataloader",
           "configure_parallelism", "freeze_unconfigured_models", "move_to_devices", "train_configured_models",
           "BatchValidationCallback", "CheckpointHook", "DDPHook", "EMAHook", "FusedGradAllReduceHook",
           "GradientAccumulationHook", "MixedPrecisionHook", "FineTuningStrategy"]

_LAZY = {"CheckpointHook": "hooks", "DDPHook": "hooks", "EMAHook": "hooks", "FusedGradAllReduceHook": "hooks",
         "GradientAccumulationHook": "hooks", "MixedPrecisionHook": "hooks", "GradientClipHook": "hooks",
         "LossSpikeSkipHook": "hooks", "ModulePatchHook": "hooks", "TrainableParameterHook": "hooks",
         "TrainingUpdateOrchestrator": "hooks", "FineTuningStrategy": "finetune"}


def __getattr__(name: str):
    import importlib

    if name in _LAZY:
        return getattr(importlib.import_module(f"nvalchemi_toolkit_b200.training.{_LAZY[name]}"), name)
    raise AttributeError(name)
