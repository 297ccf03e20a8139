# SPDX-License-Identifier: Apache-2.0
"""Time-unit conversion: public API in fs, kernels in sqrt(amu*A^2/eV).

Constants as in the reference (``nvalchemi/dynamics/_units.py:21-31``,
``dynamics/hooks/_utils.py:45``).
"""
FS_PER_INTERNAL_TIME: float = 10.180505710759414
KB_EV: float = 8.617333262e-5


def fs_to_internal_time(value):
    return value / FS_PER_INTERNAL_TIME


def per_fs_to_internal_rate(value):
    return value * FS_PER_INTERNAL_TIME
