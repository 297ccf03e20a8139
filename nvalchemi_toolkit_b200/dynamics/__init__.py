# SPDX-License-Identifier: Apache-2.0
"""Dynamics: integrators, optimisers, stage fusion, pipelining, inflight batching."""
from nvalchemi_toolkit_b200.dynamics.base import (
    BaseDynamics, BufferConfig, ConvergenceHook, DynamicsStage, FusedStage,
)
from nvalchemi_toolkit_b200.dynamics.demo import DemoDynamics
from nvalchemi_toolkit_b200.dynamics.integrators import NVE, NVTLangevin
from nvalchemi_toolkit_b200.dynamics.optimizers import FIRE

from nvalchemi_toolkit_b200.hooks.core import Hook

__all__ = ["BaseDynamics", "BufferConfig", "ConvergenceHook", "DynamicsStage", "FusedStage", "DemoDynamics", "NVE",
           "NVTLangevin", "FIRE", "Hook", "DistributedPipeline", "SizeAwareSampler", "DataSink", "GPUBuffer", "HostMemory",
           "ZarrData", "NVTNoseHoover", "NPT", "NPH", "FIRE2", "FIREVariableCell", "FIRE2VariableCell",
           "initialize_velocities", "hooks", "integrators", "optimizers"]


def __getattr__(name: str):
    import importlib

    lazy = {"DistributedPipeline": "nvalchemi_toolkit_b200.dynamics.pipeline",
            "SizeAwareSampler": "nvalchemi_toolkit_b200.dynamics.sampler",
            "DataSink": "nvalchemi_toolkit_b200.dynamics.sinks", "GPUBuffer": "nvalchemi_toolkit_b200.dynamics.sinks",
            "HostMemory": "nvalchemi_toolkit_b200.dynamics.sinks", "ZarrData": "nvalchemi_toolkit_b200.dynamics.sinks",
            "NVTNoseHoover": "nvalchemi_toolkit_b200.dynamics.integrators.nvt_nose_hoover",
            "NPT": "nvalchemi_toolkit_b200.dynamics.integrators.npt", "NPH": "nvalchemi_toolkit_b200.dynamics.integrators.nph",
            "FIRE2": "nvalchemi_toolkit_b200.dynamics.optimizers.fire2",
            "FIREVariableCell": "nvalchemi_toolkit_b200.dynamics.optimizers.fire_cell",
            "FIRE2VariableCell": "nvalchemi_toolkit_b200.dynamics.optimizers.fire2"}
    if name in lazy:
        return getattr(importlib.import_module(lazy[name]), name)
    if name == "initialize_velocities":
        from nvalchemi_toolkit_b200.dynamics._ops import initialize_velocities

        return initialize_velocities
    if name in ("hooks", "integrators", "optimizers", "sinks", "sampler", "pipeline"):
        return importlib.import_module(f"nvalchemi_toolkit_b200.dynamics.{name}")
    raise AttributeError(name)
