# SPDX-License-Identifier: Apache-2.0
"""Compressed, sharded Zarr v3 stores: many chunks and their offset index live in one shard file, which keeps the file
count of large datasets small; chunks are Zstandard-compressed.  Written and read without the ``zarr`` package."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.data.zarr_store import (AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig,
                                                    ZarrWriteConfig)

data = [systems.argon_cluster(8 + i % 7, noise=0.1, seed=i) for i in range(200)]
root = Path(tempfile.mkdtemp())
plain = ZarrWriteConfig(core=ZarrArrayConfig(chunk_rows=64), meta=ZarrArrayConfig(chunk_rows=64))
packed = ZarrWriteConfig(core=ZarrArrayConfig(chunk_rows=64, shard_rows=1024, compressor="zstd"),
                         meta=ZarrArrayConfig(chunk_rows=64, shard_rows=1024))
for name, cfg in (("plain", plain), ("sharded", packed)):
    AtomicDataZarrWriter(root / name, cfg).write(data)
    files = [f for f in (root / name).rglob("*") if f.is_file()]
    size = sum(f.stat().st_size for f in files)
    reader = AtomicDataZarrReader(root / name)
    sample, meta = reader.read(17)
    assert torch.allclose(sample["positions"], data[17].positions)
    print(f"{name:8s}: {len(files):4d} files, {size / 1024:7.1f} KiB, {len(reader)} samples, sample 17 has {meta[0] if isinstance(meta, tuple) else sample['positions'].shape[0]} atoms")
