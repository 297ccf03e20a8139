# SPDX-License-Identifier: Apache-2.0
"""Model wrappers implementing the ``BaseModelMixin`` contract."""
from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat
from nvalchemi_toolkit_b200.models.demo import DemoModel, DemoModelWrapper

__all__ = ["BaseModelMixin", "ModelConfig", "NeighborConfig", "NeighborListFormat", "DemoModel", "DemoModelWrapper"]


def __getattr__(name: str):
    import importlib

    lazy = {"LennardJonesModelWrapper": "lj", "DFTD3ModelWrapper": "dftd3", "EwaldModelWrapper": "ewald",
            "PMEModelWrapper": "pme", "MACEWrapper": "mace", "MACE": "mace", "MACEConfig": "mace", "PipelineModelWrapper": "pipeline",
            "PipelineGroup": "pipeline", "PipelineStep": "pipeline", "AIMNet2Wrapper": "aimnet2", "UMAWrapper": "uma"}
    if name in lazy:
        return getattr(importlib.import_module(f"nvalchemi_toolkit_b200.models.{lazy[name]}"), name)
    raise AttributeError(name)
