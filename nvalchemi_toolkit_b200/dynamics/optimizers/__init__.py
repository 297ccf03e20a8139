# SPDX-License-Identifier: Apache-2.0
from nvalchemi_toolkit_b200.dynamics.optimizers.fire import FIRE

__all__ = ["FIRE"]
