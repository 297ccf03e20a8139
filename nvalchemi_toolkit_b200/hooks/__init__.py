# SPDX-License-Identifier: Apache-2.0
"""Hook system shared by dynamics and training engines."""
from nvalchemi_toolkit_b200.hooks.core import (
    CheckpointableHook, DynamicsContext, Hook, HookContext, HookRegistryMixin, TrainContext,
)

_REPORTING = ("Reporter", "ReporterMessage", "ReportingErrorPolicy", "ReportingOrchestrator", "ReportingState", "RichLayout",
              "RichReporter", "ScalarCallback", "ScalarSnapshot", "TensorBoardReporter", "TensorBoardWriter", "JSONLReporter",
              "collect_scalars", "extract_dynamics_scalars", "extract_loss_scalars", "extract_optimizer_lr_scalars",
              "extract_progress_scalars", "extract_scalars", "reduce_scalars_across_ranks", "text_plot", "resolve_layout")
#: layout classes under the names the reference exports them (``hooks/reporting/layouts``)
_LAYOUT_ALIASES = {"BaseRichLayout": "BaseDashboardLayout", "DynamicsRichLayout": "DynamicsLayout",
                   "TrainingRichLayout": "TrainingLayout", "CompactRichLayout": "CompactLayout"}

__all__ = ["CheckpointableHook", "DynamicsContext", "Hook", "HookContext", "HookRegistryMixin", "TrainContext",
           "NeighborListHook", "WrapPeriodicHook", "BiasedPotentialHook", "StageTimingHook", "TorchProfilerHook",
           *_REPORTING, *_LAYOUT_ALIASES]


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
    if name in _REPORTING:
        return getattr(importlib.import_module("nvalchemi_toolkit_b200.hooks.reporting"), name)
    if name in _LAYOUT_ALIASES:
        return getattr(importlib.import_module("nvalchemi_toolkit_b200.hooks.reporting"), _LAYOUT_ALIASES[name])
    raise AttributeError(name)
