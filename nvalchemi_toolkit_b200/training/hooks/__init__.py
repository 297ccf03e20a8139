# SPDX-License-Identifier: Apache-2.0
"""Training hooks (reference ``nvalchemi/training/hooks``)."""
from nvalchemi_toolkit_b200.training.hooks.library import (
    CheckpointHook, DDPHook, EMAHook, FusedGradAllReduceHook, GradientAccumulationHook, GradientClipHook,
    LossSpikeSkipHook, MixedPrecisionHook, ModulePatchHook, TrainableParameterHook, TrainingUpdateHook,
    TrainingUpdateOrchestrator,
)
from nvalchemi_toolkit_b200.hooks.profiling import TorchProfilerHook

__all__ = ["CheckpointHook", "DDPHook", "EMAHook", "FusedGradAllReduceHook", "GradientAccumulationHook",
           "GradientClipHook", "LossSpikeSkipHook", "MixedPrecisionHook", "ModulePatchHook", "TrainableParameterHook",
           "TrainingUpdateOrchestrator", "TrainingUpdateHook", "TorchProfilerHook"]
