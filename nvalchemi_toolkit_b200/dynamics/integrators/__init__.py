# SPDX-License-Identifier: Apache-2.0
from nvalchemi_toolkit_b200.dynamics.integrators.nve import NVE
from nvalchemi_toolkit_b200.dynamics.integrators.nvt_langevin import NVTLangevin

__all__ = ["NVE", "NVTLangevin"]
