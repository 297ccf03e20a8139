# SPDX-License-Identifier: Apache-2.0
"""The 18 training stages (names and order of the reference, ``nvalchemi/training/_stages.py:105-122``).

``DO_BACKWARD`` and ``DO_OPTIMIZER_STEP`` are claim slots: when a hook subscribes to one of them it replaces the
strategy's default ``loss.backward()`` / ``optimizer.step()``; at most one hook may claim each."""
from enum import Enum, auto


class TrainingStage(Enum):
    SETUP = auto()
    BEFORE_TRAINING = auto()
    BEFORE_EPOCH = auto()
    BEFORE_BATCH = auto()
    BEFORE_FORWARD = auto()
    AFTER_FORWARD = auto()
    BEFORE_LOSS = auto()
    AFTER_LOSS = auto()
    BEFORE_BACKWARD = auto()
    DO_BACKWARD = auto()
    AFTER_BACKWARD = auto()
    BEFORE_OPTIMIZER_STEP = auto()
    DO_OPTIMIZER_STEP = auto()
    AFTER_OPTIMIZER_STEP = auto()
    AFTER_BATCH = auto()
    AFTER_EPOCH = auto()
    AFTER_TRAINING = auto()
    AFTER_VALIDATION = auto()
