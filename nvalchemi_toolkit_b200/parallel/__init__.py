# SPDX-License-Identifier: Apache-2.0
"""Multi-GPU plumbing: symmetric (peer-mapped) memory arenas, device-side barriers, fused P2P collectives."""
from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext, SymmetricArena

__all__ = ["P2PContext", "SymmetricArena"]
