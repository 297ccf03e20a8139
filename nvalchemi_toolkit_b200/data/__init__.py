# SPDX-License-Identifier: Apache-2.0
"""Data layer: ``AtomicData``, ``Batch``, columnar storages, datapipes and Zarr IO."""
from nvalchemi_toolkit_b200.data.atomic_data import AtomicData, DataMixin
from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.level_storage import (
    LevelSchema, MultiLevelStorage, SegmentedLevelStorage, UniformLevelStorage,
)

__all__ = ["AtomicData", "Batch", "DataMixin", "LevelSchema", "MultiLevelStorage", "SegmentedLevelStorage",
           "UniformLevelStorage", "AtomicDataZarrReader", "AtomicDataZarrWriter", "BatchDatasetProtocol", "Compose",
           "DataLoader", "Dataset", "InMemoryDataset", "MultiDataset", "Reader", "transforms"]

_LAZY = {"AtomicDataZarrReader": "zarr_store", "AtomicDataZarrWriter": "zarr_store", "ZarrWriteConfig": "zarr_store",
         "ZarrArrayConfig": "zarr_store", "BatchDatasetProtocol": "datapipes", "Compose": "transforms", "DataLoader": "datapipes",
         "Dataset": "datapipes", "InMemoryDataset": "datapipes", "MultiDataset": "datapipes", "Reader": "datapipes",
         "MultiDatasetSampler": "datapipes", "MultiDatasetBatchSampler": "datapipes", "FixedCompositionBatchSampler": "datapipes"}


def __getattr__(name: str):  # datapipes and Zarr IO load on first use
    import importlib

    if name in ("transforms", "datapipes", "zarr_store"):
        return importlib.import_module(f"nvalchemi_toolkit_b200.data.{name}")
    if name in _LAZY:
        return getattr(importlib.import_module(f"nvalchemi_toolkit_b200.data.{_LAZY[name]}"), name)
    raise AttributeError(name)
