# SPDX-License-Identifier: Apache-2.0
"""Dynamics hooks: safety, monitoring, constraints, snapshots, logging (reference ``nvalchemi/dynamics/hooks``)."""
from nvalchemi_toolkit_b200.dynamics.hooks.library import (
    AlignCellHook, ConvergedSnapshotHook, EnergyDriftMonitorHook, FreezeAtomsHook, LoggingHook, MaxForceClampHook,
    NaNDetectorHook, SnapshotHook,
)

from nvalchemi_toolkit_b200.hooks.profiling import TorchProfilerHook
from nvalchemi_toolkit_b200.hooks.stage_timing import StageTimingHook

__all__ = ["AlignCellHook", "ConvergedSnapshotHook", "EnergyDriftMonitorHook", "FreezeAtomsHook", "LoggingHook",
           "MaxForceClampHook", "NaNDetectorHook", "SnapshotHook", "StageTimingHook", "TorchProfilerHook"]
