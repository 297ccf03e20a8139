# SPDX-License-Identifier: Apache-2.0
"""Data layer: ``AtomicData``, ``Batch``, columnar storages, datapipes and Zarr IO."""
from nvalchemi_toolkit_b200.data.atomic_data import AtomicData, DataMixin
from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.level_storage import (
    LevelSchema, MultiLevelStorage, SegmentedLevelStorage, UniformLevelStorage,
)

__all__ = ["AtomicData", "Batch", "DataMixin", "LevelSchema", "MultiLevelStorage", "SegmentedLevelStorage",
           "UniformLevelStorage"]
