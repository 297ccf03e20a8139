# SPDX-License-Identifier: Apache-2.0
"""Operator layer: thin Python entry points over the sm_100a extension with torch CPU paths."""
from nvalchemi_toolkit_b200.ops import _native  # noqa: F401
