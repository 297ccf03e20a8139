# SPDX-License-Identifier: Apache-2.0
"""``NPH`` lives with ``NPT`` (shared MTK machinery); this module keeps the reference's import path."""
from nvalchemi_toolkit_b200.dynamics.integrators.npt import NPH  # noqa: F401
