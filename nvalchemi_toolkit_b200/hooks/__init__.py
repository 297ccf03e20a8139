# SPDX-License-Identifier: Apache-2.0
"""Hook system shared by dynamics and training engines."""
from nvalchemi_toolkit_b200.hooks.core import (
    CheckpointableHook, DynamicsContext, Hook, HookContext, HookRegistryMixin, TrainContext,
)

__all__ = ["CheckpointableHook", "DynamicsContext", "Hook", "HookContext", "HookRegistryMixin", "TrainContext"]


def __getattr__(name: str):  # lazy: these import models/dynamics
    import importlib

    lazy = {
        "NeighborListHook": "nvalchemi_toolkit_b200.hooks.neighbor_list",
        "WrapPeriodicHook": "nvalchemi_toolkit_b200.hooks.periodic",
        "BiasedPotentialHook": "nvalchemi_toolkit_b200.hooks.bias",
        "StageTimingHook": "nvalchemi_toolkit_b200.hooks.stage_timing",
        "TorchProfilerHook": "nvalchemi_toolkit_b200.hooks.profiling",
    }
    if name in lazy:
        return getattr(importlib.import_module(lazy[name]), name)
    raise AttributeError(name)
