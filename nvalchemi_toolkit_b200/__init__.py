# SPDX-License-Identifier: Apache-2.0
"""B200-native atomistic simulation and MLIP training framework.

Capabilities follow NVIDIA's ``nvalchemi-toolkit`` (package ``nvalchemi`` 0.1.0); the compute
path is PyTorch plus hand-written sm_100a CUDA kernels (``torch.ops.nvalchemi.*``) and
NVLink peer-to-peer communication kernels.
"""
__version__ = "0.1.0"
version = __version__  # the reference package spells it this way

from nvalchemi_toolkit_b200._optional import MissingDependencyError, OptionalDependency  # noqa: F401
from nvalchemi_toolkit_b200._typing import AtomCategory  # noqa: F401
from nvalchemi_toolkit_b200.data import AtomicData, Batch  # noqa: F401
from nvalchemi_toolkit_b200.ops import compat as _compat  # noqa: F401,E402  registers the reference's operator names

OptionalDependencyError = MissingDependencyError  # the reference's name for the same error
