# SPDX-License-Identifier: Apache-2.0
"""Write structures to a Zarr v3 store, read them back, and iterate size-balanced batches."""
import tempfile
from pathlib import Path

import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.data.datapipes import DataLoader, Dataset
from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig, ZarrWriteConfig

store = Path(tempfile.mkdtemp()) / "clusters.zarr"
data = [systems.argon_cluster(n, seed=n) for n in range(10, 40, 3)]
writer = AtomicDataZarrWriter(store, ZarrWriteConfig(core=ZarrArrayConfig(chunk_rows=256, compressor="gzip")))
writer.append(Batch.from_data_list(data[:5]))
writer.append(Batch.from_data_list(data[5:]))
writer.add_custom("temperature_K", torch.linspace(100, 300, len(data)), level="system")
reader = AtomicDataZarrReader(store)
print(len(reader), "samples; atoms/edges of sample 3:", reader.get_metadata(3))
sample, meta = reader.read(3)
print("fields:", sorted(sample)[:6], "...")
loader = DataLoader(Dataset(reader), batch_size=4, shuffle=True, seed=0)
for epoch in range(2):
    loader.set_epoch(epoch)
    print(f"epoch {epoch}:", [b.num_nodes_list for b in loader])
writer.delete([0, 1])
reader.refresh()
print("after deleting two samples:", len(reader), "live of", reader.num_total, "stored")
