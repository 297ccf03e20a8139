# SPDX-License-Identifier: Apache-2.0
"""Native MACE: network, O(3) tables and the ``BaseModelMixin`` wrapper."""
from nvalchemi_toolkit_b200.models.mace.model import MACE, MACEConfig
from nvalchemi_toolkit_b200.models.mace.wrapper import MACEWrapper

__all__ = ["MACE", "MACEConfig", "MACEWrapper"]
