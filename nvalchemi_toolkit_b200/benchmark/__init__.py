# SPDX-License-Identifier: Apache-2.0
"""Benchmark suite: synthetic systems and config-driven forward / NVT runners
(``python -m nvalchemi_toolkit_b200.benchmark.runners <config.yaml>``; under ``torchrun`` for domain decomposition)."""
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.benchmark.systems import SYSTEMS, build

__all__ = ["systems", "SYSTEMS", "build"]
