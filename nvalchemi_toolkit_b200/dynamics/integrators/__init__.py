# SPDX-License-Identifier: Apache-2.0
"""Integrators: NVE, NVT (Langevin, Nose-Hoover chains), NPT and NPH (Martyna-Tobias-Klein)."""
from nvalchemi_toolkit_b200.dynamics.integrators.nve import NVE
from nvalchemi_toolkit_b200.dynamics.integrators.nvt_langevin import NVTLangevin

__all__ = ["NVE", "NVTLangevin", "NVTNoseHoover", "NPT", "NPH"]

_LAZY = {"NVTNoseHoover": "nvt_nose_hoover", "NPT": "npt", "NPH": "nph"}


def __getattr__(name: str):
    import importlib

    if name in _LAZY:
        return getattr(importlib.import_module(f"nvalchemi_toolkit_b200.dynamics.integrators.{_LAZY[name]}"), name)
    raise AttributeError(name)
