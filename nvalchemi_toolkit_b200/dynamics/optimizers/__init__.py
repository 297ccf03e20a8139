# SPDX-License-Identifier: Apache-2.0
"""Geometry optimisers: FIRE, FIRE2 and their variable-cell forms."""
from nvalchemi_toolkit_b200.dynamics.optimizers.fire import FIRE

__all__ = ["FIRE", "FIRE2", "FIREVariableCell", "FIRE2VariableCell"]

_LAZY = {"FIRE2": "fire2", "FIRE2VariableCell": "fire2", "FIREVariableCell": "fire_cell"}


def __getattr__(name: str):
    import importlib

    if name in _LAZY:
        return getattr(importlib.import_module(f"nvalchemi_toolkit_b200.dynamics.optimizers.{_LAZY[name]}"), name)
    raise AttributeError(name)
