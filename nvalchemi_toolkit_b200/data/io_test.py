# SPDX-License-Identifier: Apache-2.0
"""``python -m nvalchemi_toolkit_b200.data.io_test {roundtrip,read}``: synthetic-data IO benchmark of the Zarr store.

Counterpart of the reference's ``nvalchemi-io-test`` command (``nvalchemi/data/io_test.py:73-1312``): generate structures
with a planned size distribution, write them under a storage configuration (codec, level, chunk and shard sizes, separate
sizes for the edge arrays), report raw size, size on disk, compression ratio, file count and write throughput, read the
store back (per sample, in DataLoader batches, sequential / shuffled / block-shuffled order, optionally into pinned
memory) with read throughput, and verify the first and last sample bit for bit.  ``--samples`` may be repeated to
sweep dataset sizes; ``read`` benchmarks an existing store.  ``argparse`` instead of click, a plain-text table plus one
JSON document on stdout.
"""
from __future__ import annotations

import argparse
import json
import shutil
import tempfile
import time
from pathlib import Path
from typing import Any, Iterator, Sequence

import torch

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData
from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.data.datapipes import DataLoader, Dataset
from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig, ZarrWriteConfig

EDGE_FIELDS = ("neighbor_list", "shifts", "unit_shifts")
READ_MODES = ("sample", "batch")
READ_ORDERS = ("sequential", "shuffle", "block-shuffle")


# ---- data -------------------------------------------------------------------------------------------------------
def plan_sizes(n: int, min_atoms: int, max_atoms: int, edges_per_atom: int, seed: int) -> list[tuple[int, int]]:
    """``(atoms, edges)`` of every structure, drawn up front so that sizes can be estimated before anything is built."""
    g = torch.Generator().manual_seed(seed)
    atoms = torch.randint(min_atoms, max_atoms + 1, (n,), generator=g).tolist()
    return [(a, a * edges_per_atom) for a in atoms]


def make_structure(num_atoms: int, num_edges: int, g: torch.Generator) -> AtomicData:
    kw: dict[str, Any] = dict(
        atomic_numbers=torch.randint(1, 90, (num_atoms,), generator=g), positions=torch.randn(num_atoms, 3, generator=g) * 5,
        forces=torch.randn(num_atoms, 3, generator=g), energy=torch.randn(1, 1, generator=g), cell=torch.eye(3) * 20,
        pbc=torch.tensor([True, True, True]))
    if num_edges:
        kw["neighbor_list"] = torch.randint(0, num_atoms, (num_edges, 2), generator=g)
        kw["shifts"] = torch.randint(-1, 2, (num_edges, 3), generator=g).to(torch.float32) * 20.0
    return AtomicData(**kw)


def synthetic(n: int, min_atoms: int, max_atoms: int, seed: int = 0, edges_per_atom: int = 0) -> list[AtomicData]:
    g = torch.Generator().manual_seed(seed + 1)
    return [make_structure(a, e, g) for a, e in plan_sizes(n, min_atoms, max_atoms, edges_per_atom, seed)]


def tensor_bytes(data: Sequence[AtomicData]) -> int:
    return sum(v.numel() * v.element_size() for d in data for v in d._tensor_items().values())


def estimate_bytes(plan: Sequence[tuple[int, int]]) -> int:
    """Uncompressed size implied by a plan: int64 numbers, three float32 vectors per atom, int64 pairs + float32 shifts per
    edge, and the per-system scalars."""
    return sum(a * (8 + 4 * 3 * 2) + e * (8 * 2 + 4 * 3) + (4 + 36 + 3) for a, e in plan)


def fmt_bytes(n: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024.0 or unit == "TiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024.0
    return f"{n:.1f} TiB"


# ---- storage configuration ----------------------------------------------------------------------------------------
def build_config(args: argparse.Namespace) -> tuple[ZarrWriteConfig, str]:
    core = ZarrArrayConfig(chunk_rows=args.chunk_size or 65536, compressor=args.compressor, level=args.level,
                           shard_rows=args.shard_size)
    overrides = {}
    if args.edge_chunk_size or args.edge_shard_size:
        edge = ZarrArrayConfig(chunk_rows=args.edge_chunk_size or core.chunk_rows, compressor=args.compressor, level=args.level,
                               shard_rows=args.edge_shard_size if args.edge_shard_size else args.shard_size)
        overrides = {k: edge for k in EDGE_FIELDS}
    cfg = ZarrWriteConfig(core=core, meta=ZarrArrayConfig(chunk_rows=16384, compressor=args.compressor, level=args.level),
                          field_overrides=overrides)
    desc = (f"codec={args.compressor or 'none'}" + (f" level={args.level}" if args.compressor else "")
            + f" chunk={core.chunk_rows}" + (f" shard={core.shard_rows}" if core.shard_rows else "")
            + (f" edge-chunk={args.edge_chunk_size}" if args.edge_chunk_size else "")
            + (f" edge-shard={args.edge_shard_size}" if args.edge_shard_size else ""))
    return cfg, desc


def dir_size(path: Path) -> int:
    return sum(f.stat().st_size for f in path.rglob("*") if f.is_file())


def file_count(path: Path) -> int:
    return sum(1 for f in path.rglob("*") if f.is_file())


# ---- reading ------------------------------------------------------------------------------------------------------
def read_indices(n: int, order: str, seed: int, block: int) -> list[int]:
    """Sample order of a read pass: as stored, fully shuffled, or shuffled in contiguous blocks of ``block`` samples (the
    blocks are permuted, samples inside a block stay in storage order: a shard-friendly shuffle)."""
    if order == "sequential":
        return list(range(n))
    g = torch.Generator().manual_seed(seed)
    if order == "shuffle":
        return torch.randperm(n, generator=g).tolist()
    if order == "block-shuffle":
        blocks = [list(range(lo, min(lo + block, n))) for lo in range(0, n, block)]
        return [i for b in torch.randperm(len(blocks), generator=g).tolist() for i in blocks[b]]
    raise ValueError(f"unknown read order {order!r}; expected one of {READ_ORDERS}")


def _batches(indices: Sequence[int], size: int) -> Iterator[list[int]]:
    for lo in range(0, len(indices), size):
        yield list(indices[lo: lo + size])


def read_pass(reader: AtomicDataZarrReader, mode: str, order: str, *, batch_size: int, prefetch: int, seed: int, block: int,
              pin_memory: bool) -> dict[str, Any]:
    """One timed pass over the whole store.  ``sample``: one backend read per structure; ``batch``: DataLoader batches of
    ``batch_size`` structures, ``prefetch`` batches fused into each backend read."""
    idx = read_indices(len(reader), order, seed, block)
    atoms = nbytes = 0
    t0 = time.perf_counter()
    if mode == "sample":
        for i in idx:
            raw = reader.read_raw(i)
            if pin_memory:
                raw = {k: v.pin_memory() for k, v in raw.items()} if torch.cuda.is_available() else raw
            atoms += int(raw["positions"].shape[0])
            nbytes += sum(v.numel() * v.element_size() for v in raw.values())
    elif mode == "batch":
        loader = DataLoader(Dataset(reader, raw=True), batch_size=batch_size, prefetch_factor=prefetch,
                            batch_sampler=list(_batches(idx, batch_size)))
        for b in loader:
            if pin_memory and torch.cuda.is_available():
                b = b.pin_memory()
            atoms += b.num_nodes
            nbytes += sum(v.numel() * v.element_size() for _, v in b._storage.items())
    else:
        raise ValueError(f"unknown read mode {mode!r}; expected one of {READ_MODES}")
    dt = time.perf_counter() - t0
    return {"mode": mode, "order": order, "samples": len(idx), "atoms": atoms, "seconds": dt,
            "samples_per_s": len(idx) / max(dt, 1e-12), "read_MBps": nbytes / 1e6 / max(dt, 1e-12)}


def expand(values: Sequence[str], all_values: Sequence[str]) -> list[str]:
    out: list[str] = []
    for v in values:
        out.extend(all_values if v in ("both", "all") else [v])
    return list(dict.fromkeys(out))


def verify(reader: AtomicDataZarrReader, data: Sequence[AtomicData]) -> bool:
    """First and last structure come back bit for bit (positions, numbers, forces, edges when present)."""
    for i in (0, len(data) - 1):
        got, want = reader.read(i)[0], data[i]
        for k in ("positions", "atomic_numbers", "forces", "neighbor_list"):
            ref = getattr(want, k, None)
            if ref is None:
                continue
            if k not in got or not torch.equal(got[k].to(ref.dtype), ref):
                return False
    return True


# ---- commands -----------------------------------------------------------------------------------------------------
def run_roundtrip(args: argparse.Namespace, n_samples: int) -> dict[str, Any]:
    plan = plan_sizes(n_samples, args.min_atoms, args.max_atoms, args.edges_per_atom, args.seed)
    data = synthetic(n_samples, args.min_atoms, args.max_atoms, args.seed, args.edges_per_atom)
    raw_bytes = tensor_bytes(data)
    keep = args.output_dir is not None
    root = Path(args.output_dir or tempfile.mkdtemp(prefix="nva_io_")) / f"store_{n_samples}.zarr"
    if root.exists():
        shutil.rmtree(root)
    cfg, desc = build_config(args)
    writer = AtomicDataZarrWriter(root, cfg)
    t0 = time.perf_counter()
    for lo in range(0, len(data), args.write_batch):
        writer.append(Batch.from_data_list(data[lo: lo + args.write_batch]))
    t_write = time.perf_counter() - t0
    reader = AtomicDataZarrReader(root)
    disk = dir_size(root)
    reads = [read_pass(reader, m, o, batch_size=args.read_batch_size, prefetch=args.read_prefetch, seed=args.read_seed,
                       block=args.read_block_size, pin_memory=args.pin_memory)
             for m in expand(args.read_mode, READ_MODES) for o in expand(args.read_order, READ_ORDERS)]
    res = {"samples": n_samples, "atoms": sum(a for a, _ in plan), "edges": sum(e for _, e in plan), "config": desc,
           "estimated_raw_bytes": estimate_bytes(plan), "raw_bytes": raw_bytes, "disk_bytes": disk,
           "compression_ratio": raw_bytes / max(disk, 1), "files": file_count(root), "write_seconds": t_write,
           "write_MBps": raw_bytes / 1e6 / max(t_write, 1e-12), "reads": reads, "roundtrip_ok": verify(reader, data),
           "store": str(root) if keep else None}
    if not keep:
        shutil.rmtree(root.parent, ignore_errors=True)
    return res


def run_read(args: argparse.Namespace) -> dict[str, Any]:
    reader = AtomicDataZarrReader(args.store)
    reads = [read_pass(reader, m, o, batch_size=args.read_batch_size, prefetch=args.read_prefetch, seed=args.read_seed,
                       block=args.read_block_size, pin_memory=args.pin_memory)
             for m in expand(args.read_mode, READ_MODES) for o in expand(args.read_order, READ_ORDERS)]
    return {"store": str(args.store), "samples": len(reader), "disk_bytes": dir_size(Path(args.store)),
            "files": file_count(Path(args.store)), "reads": reads}


def print_results(results: Sequence[dict[str, Any]]) -> None:
    for r in results:
        if "raw_bytes" in r:
            print(f"{r['samples']:>8} samples  {r['config']}")
            print(f"         raw {fmt_bytes(r['raw_bytes'])} (estimated {fmt_bytes(r['estimated_raw_bytes'])})  on disk "
                  f"{fmt_bytes(r['disk_bytes'])}  ratio {r['compression_ratio']:.2f}x  files {r['files']}  "
                  f"write {r['write_MBps']:.1f} MB/s  round trip {'ok' if r['roundtrip_ok'] else 'MISMATCH'}")
        else:
            print(f"{r['samples']:>8} samples in {r['store']}: {fmt_bytes(r['disk_bytes'])} on disk, {r['files']} files")
        for p in r["reads"]:
            print(f"         read {p['mode']:<6} {p['order']:<13} {p['samples_per_s']:>10.1f} samples/s  {p['read_MBps']:>8.1f} MB/s")


def _add_read_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--read-mode", action="append", choices=list(READ_MODES) + ["both"], default=None,
                   help="per-sample reads, DataLoader batches, or both (repeatable)")
    p.add_argument("--read-batch-size", type=int, default=64, help="samples per DataLoader batch for --read-mode batch")
    p.add_argument("--read-prefetch", type=int, default=4, help="DataLoader batches fused into each backend read")
    p.add_argument("--read-order", action="append", choices=list(READ_ORDERS) + ["all"], default=None,
                   help="sequential, shuffle or block-shuffle (repeatable)")
    p.add_argument("--read-seed", type=int, default=0, help="seed of the shuffled orders")
    p.add_argument("--read-block-size", type=int, default=256, help="contiguous block of --read-order block-shuffle")
    p.add_argument("--pin-memory", action="store_true", help="read into pinned host memory (when a GPU is present)")


def main(argv: list[str] | None = None) -> Any:
    ap = argparse.ArgumentParser(prog="nvalchemi-io-test", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd")
    a = sub.add_parser("roundtrip", help="generate, write, read back, verify (the default command)")
    a.add_argument("--samples", "-n", type=int, action="append", default=None, help="number of systems (repeat to sweep)")
    a.add_argument("--min-atoms", type=int, default=8)
    a.add_argument("--max-atoms", type=int, default=64)
    a.add_argument("--edges-per-atom", type=int, default=0, help="synthetic neighbour-list edges per atom (0: no edge arrays)")
    a.add_argument("--compressor", "--codec", default=None, choices=[None, "gzip", "zstd"], help="omit for no compression")
    a.add_argument("--level", type=int, default=3)
    a.add_argument("--chunk-size", "--chunk-rows", type=int, default=None, help="rows per chunk (omit for the store's default)")
    a.add_argument("--shard-size", type=int, default=None, help="rows per shard file (omit for one file per chunk)")
    a.add_argument("--edge-chunk-size", type=int, default=None, help="rows per chunk of neighbor_list / shifts")
    a.add_argument("--edge-shard-size", type=int, default=None, help="rows per shard of neighbor_list / shifts")
    a.add_argument("--seed", type=int, default=0)
    a.add_argument("--write-batch", type=int, default=256, help="systems per append call")
    a.add_argument("--output-dir", "--store", default=None, help="keep the stores here (default: temporary, removed)")
    _add_read_options(a)
    b = sub.add_parser("read", help="read benchmark of an existing store")
    b.add_argument("store")
    _add_read_options(b)
    argv = list(argv) if argv is not None else None
    import sys

    raw = sys.argv[1:] if argv is None else argv
    if not raw or raw[0] not in ("roundtrip", "read", "-h", "--help"):
        raw = ["roundtrip"] + list(raw)  # options without a command mean roundtrip, as in the reference tool
    args = ap.parse_args(raw)
    args.read_mode = args.read_mode or ["batch"]
    args.read_order = args.read_order or ["sequential"]
    if args.cmd == "read":
        results = [run_read(args)]
    else:
        results = [run_roundtrip(args, n) for n in (args.samples or [1000])]
    print_results(results)
    print(json.dumps(results if len(results) > 1 else results[0], indent=1))
    return results if len(results) > 1 else results[0]


if __name__ == "__main__":
    main()
