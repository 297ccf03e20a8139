# SPDX-License-Identifier: Apache-2.0
"""``python -m nvalchemi_toolkit_b200.data.io_test {roundtrip,read}``: synthetic-data IO benchmark of the Zarr store
(write / read throughput, compression ratio, file count).  Counterpart of the reference's ``nvalchemi-io-test`` CLI
(``nvalchemi/data/io_test.py:73-1312``); ``argparse`` instead of click, plain-text report."""
from __future__ import annotations

import argparse
import json
import shutil
import tempfile
import time
from pathlib import Path

import torch

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData
from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.datapipes import DataLoader, Dataset
from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig, ZarrWriteConfig


def synthetic(n: int, min_atoms: int, max_atoms: int, seed: int = 0) -> list[AtomicData]:
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        k = int(torch.randint(min_atoms, max_atoms + 1, (1,), generator=g))
        out.append(AtomicData(atomic_numbers=torch.randint(1, 90, (k,), generator=g),
                              positions=torch.randn(k, 3, generator=g) * 5, forces=torch.randn(k, 3, generator=g),
                              energy=torch.randn(1, 1, generator=g), cell=torch.eye(3) * 20,
                              pbc=torch.tensor([True, True, True])))
    return out


def roundtrip(args: argparse.Namespace) -> dict:
    data = synthetic(args.samples, args.min_atoms, args.max_atoms)
    raw_bytes = sum(v.numel() * v.element_size() for d in data for v in d._tensor_items().values())
    root = Path(args.store or tempfile.mkdtemp(prefix="nva_io_")) / "store.zarr"
    if root.exists():
        shutil.rmtree(root)
    cfg = ZarrWriteConfig(core=ZarrArrayConfig(chunk_rows=args.chunk_rows, compressor=args.compressor, level=args.level),
                          meta=ZarrArrayConfig(chunk_rows=16384, compressor=args.compressor, level=args.level))
    w = AtomicDataZarrWriter(root, cfg)
    t0 = time.perf_counter()
    for lo in range(0, len(data), args.write_batch):
        w.append(Batch.from_data_list(data[lo: lo + args.write_batch]))
    t_write = time.perf_counter() - t0
    r = AtomicDataZarrReader(root)
    t0 = time.perf_counter()
    n = sum(b.num_graphs for b in DataLoader(Dataset(r, raw=True), batch_size=args.batch_size, prefetch_factor=4))
    t_read = time.perf_counter() - t0
    first = r.read(0)[0]
    ok = torch.allclose(first["positions"], data[0].positions) and n == args.samples
    disk = r.nbytes_on_disk()
    files = sum(1 for f in root.rglob("*") if f.is_file())
    return {"samples": args.samples, "raw_MB": raw_bytes / 1e6, "disk_MB": disk / 1e6,
            "compression_ratio": raw_bytes / max(disk, 1), "files": files, "write_MBps": raw_bytes / 1e6 / t_write,
            "read_MBps": raw_bytes / 1e6 / t_read, "roundtrip_ok": bool(ok), "store": str(root)}


def read(args: argparse.Namespace) -> dict:
    r = AtomicDataZarrReader(args.store)
    t0 = time.perf_counter()
    atoms = 0
    for b in DataLoader(Dataset(r, raw=True), batch_size=args.batch_size, prefetch_factor=4):
        atoms += b.num_nodes
    dt = time.perf_counter() - t0
    return {"samples": len(r), "atoms": atoms, "seconds": dt, "samples_per_s": len(r) / dt}


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser(prog="nvalchemi-io-test")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("roundtrip")
    a.add_argument("--samples", type=int, default=1000)
    a.add_argument("--min-atoms", type=int, default=8)
    a.add_argument("--max-atoms", type=int, default=64)
    a.add_argument("--compressor", default=None, choices=[None, "gzip", "zstd"])
    a.add_argument("--level", type=int, default=3)
    a.add_argument("--chunk-rows", type=int, default=16384)
    a.add_argument("--write-batch", type=int, default=256)
    a.add_argument("--batch-size", type=int, default=64)
    a.add_argument("--store", default=None)
    b = sub.add_parser("read")
    b.add_argument("store")
    b.add_argument("--batch-size", type=int, default=64)
    args = ap.parse_args(argv)
    res = roundtrip(args) if args.cmd == "roundtrip" else read(args)
    print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
