# SPDX-License-Identifier: Apache-2.0
"""Zarr v3 storage of atomistic datasets, written and read without the ``zarr`` package.

On-disk layout (the reference's, ``nvalchemi/data/datapipes/backends/zarr.py:433-450,715-716``)::

    <store>/zarr.json                 group; attributes: num_samples, fields = {"core": {name: level}, "custom": {...}}
    <store>/meta/atoms_ptr            int64[N+1]   CSR offsets of atoms per sample
    <store>/meta/edges_ptr            int64[N+1]
    <store>/meta/samples_mask         bool[N]      False = soft-deleted sample
    <store>/meta/atoms_mask, edges_mask  bool[V], bool[E]
    <store>/core/<field>              concatenated over samples along axis 0 (system fields: one row per sample)
    <store>/custom/<key>              user arrays added later

Arrays are regular-chunked along axis 0 with the ``bytes`` codec (little endian), optionally followed by ``gzip`` or
``zstd`` and optionally wrapped in ``sharding_indexed`` (``ZarrArrayConfig.shard_rows``: many chunks and their offset
index in one file); each array directory holds ``zarr.json`` and chunk files ``c/<i>/0/...``.  Stores written here are
plain Zarr v3 and can be opened by ``zarr>=3``; stores written by the reference are readable with the codecs of
``data/zarr_codecs.py`` (``bytes, gzip, zstd, crc32c, blosc`` with LZ4 / Zstd / zlib and byte shuffle, ``transpose``,
``sharding_indexed``).
"""
from __future__ import annotations

import json
import os
import zlib
from pathlib import Path
from typing import Any, Sequence

import numpy as np
import torch
from pydantic import BaseModel

from nvalchemi_toolkit_b200.data import zarr_codecs as _codecs

from nvalchemi_toolkit_b200.data.level_storage import LevelSchema

_DTYPES = {"bool": np.bool_, "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64, "uint8": np.uint8,
           "float16": np.float16, "float32": np.float32, "float64": np.float64}
_NAMES = {np.dtype(v).name: k for k, v in _DTYPES.items()}


class ZarrArrayConfig(BaseModel):
    """Per-group (or per-field) storage options."""

    chunk_rows: int = 65536
    compressor: str | None = None  # None | "gzip" | "zstd"
    level: int = 3
    #: rows per shard file (a multiple of ``chunk_rows``): many chunks + an offset index in ONE file (Zarr v3
    #: ``sharding_indexed``), which keeps the file count of large datasets small.  None: one file per chunk.
    shard_rows: int | None = None


class ZarrWriteConfig(BaseModel):
    core: ZarrArrayConfig = ZarrArrayConfig()
    meta: ZarrArrayConfig = ZarrArrayConfig(chunk_rows=16384)
    custom: ZarrArrayConfig = ZarrArrayConfig()
    field_overrides: dict[str, ZarrArrayConfig] = {}


def _write_json(path: Path, obj: dict) -> None:
    tmp = path.with_suffix(".tmp")
    tmp.write_text(json.dumps(obj, indent=1))
    os.replace(tmp, path)


def _group(path: Path, attributes: dict | None = None) -> None:
    path.mkdir(parents=True, exist_ok=True)
    _write_json(path / "zarr.json", {"zarr_format": 3, "node_type": "group", "attributes": attributes or {}})


class ZarrArray:
    """One chunked array, growable along axis 0."""

    def __init__(self, path: Path) -> None:
        self.path = Path(path)
        self.meta = json.loads((self.path / "zarr.json").read_text())
        if self.meta.get("node_type") != "array":
            raise ValueError(f"{path} is not a Zarr v3 array")
        self.dtype = np.dtype(_DTYPES[self.meta["data_type"]])
        self.chunk = tuple(self.meta["chunk_grid"]["configuration"]["chunk_shape"])
        self.codecs = [c["name"] for c in self.meta["codecs"]]
        _codecs.check_supported(self.meta["codecs"])
        enc = self.meta.get("chunk_key_encoding", {"name": "default", "configuration": {"separator": "/"}})
        self.sep = enc.get("configuration", {}).get("separator", "/")
        self.prefix = "c" if enc["name"] == "default" else ""

    @classmethod
    def create(cls, path: Path, shape: Sequence[int], dtype: Any, cfg: ZarrArrayConfig) -> "ZarrArray":
        path = Path(path)
        path.mkdir(parents=True, exist_ok=True)
        name = _NAMES[np.dtype(dtype).name]
        codecs: list[dict] = [{"name": "bytes", "configuration": {"endian": "little"}}]
        if cfg.compressor == "gzip":
            codecs.append({"name": "gzip", "configuration": {"level": cfg.level}})
        elif cfg.compressor == "zstd":
            if not _codecs.zstd_available():
                raise ImportError("zstd compression needs the 'zstandard' package or pyarrow's Zstandard codec")
            codecs.append({"name": "zstd", "configuration": {"level": cfg.level, "checksum": False}})
        elif cfg.compressor is not None:
            raise ValueError(f"unknown compressor {cfg.compressor!r}")
        chunk = [max(1, int(cfg.chunk_rows))] + [max(1, int(s)) for s in shape[1:]]
        if cfg.shard_rows is not None:
            if cfg.shard_rows % chunk[0] != 0:
                raise ValueError(f"shard_rows ({cfg.shard_rows}) must be a multiple of chunk_rows ({chunk[0]})")
            codecs = [{"name": "sharding_indexed", "configuration": {
                "chunk_shape": list(chunk), "codecs": codecs, "index_location": "end",
                "index_codecs": [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "crc32c"}]}}]
            chunk = [int(cfg.shard_rows)] + chunk[1:]
        _write_json(path / "zarr.json", {
            "zarr_format": 3, "node_type": "array", "shape": [int(s) for s in shape], "data_type": name,
            "chunk_grid": {"name": "regular", "configuration": {"chunk_shape": chunk}},
            "chunk_key_encoding": {"name": "default", "configuration": {"separator": "/"}},
            "fill_value": False if name == "bool" else 0, "codecs": codecs, "attributes": {}, "dimension_names": None})
        return cls(path)

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.meta["shape"])

    def _chunk_path(self, i: int) -> Path:
        parts = [str(i)] + ["0"] * (len(self.shape) - 1)
        key = self.sep.join(([self.prefix] if self.prefix else []) + parts)
        return self.path / key

    def _decode(self, raw: bytes) -> np.ndarray:
        return _codecs.decode(raw, self.meta["codecs"], self.dtype, self.chunk)

    def _encode(self, arr: np.ndarray) -> bytes:
        return _codecs.encode(arr, self.meta["codecs"], self.dtype)

    #: decoded chunks kept per array: random per-sample reads touch the same chunk (or shard) many times, and decoding a
    #: compressed shard costs milliseconds.  Entries are validated against the file's size and modification time, so a
    #: chunk rewritten by another writer object is decoded again.
    CACHE_CHUNKS = 4

    def _read_chunk(self, i: int) -> np.ndarray:
        p = self._chunk_path(i)
        try:
            st = p.stat()
        except FileNotFoundError:
            return np.full(self.chunk, self.meta.get("fill_value", 0), dtype=self.dtype)
        cache = self.__dict__.setdefault("_chunk_cache", {})
        stamp = (st.st_size, st.st_mtime_ns)
        hit = cache.get(i)
        if hit is not None and hit[0] == stamp:
            cache[i] = cache.pop(i)  # most recently used last
            return hit[1]
        arr = self._decode(p.read_bytes())
        arr.setflags(write=False)  # shared with later readers of the same chunk
        cache[i] = (stamp, arr)
        while len(cache) > self.CACHE_CHUNKS:
            cache.pop(next(iter(cache)))
        return arr

    def read(self, start: int = 0, stop: int | None = None) -> np.ndarray:
        n = self.shape[0]
        stop = n if stop is None else min(stop, n)
        start = max(0, start)
        if stop <= start:
            return np.zeros((0,) + self.shape[1:], dtype=self.dtype)
        cr = self.chunk[0]
        parts = []
        for ci in range(start // cr, (stop - 1) // cr + 1):
            ch = self._read_chunk(ci)
            lo, hi = max(start, ci * cr) - ci * cr, min(stop, (ci + 1) * cr) - ci * cr
            parts.append(ch[lo:hi])
        tail = tuple(slice(0, s) for s in self.shape[1:])
        if len(parts) == 1:
            return np.array(parts[0][(slice(None),) + tail])  # a copy: the chunk itself stays in the cache, read-only
        return np.concatenate(parts, 0)[(slice(None),) + tail]

    def write(self, start: int, data: np.ndarray) -> None:
        """Overwrite rows ``[start, start + len(data))`` (the array must already be large enough)."""
        data = np.asarray(data, dtype=self.dtype).reshape((-1,) + self.shape[1:])
        stop = start + data.shape[0]
        cr = self.chunk[0]
        for ci in range(start // cr, (max(stop, start + 1) - 1) // cr + 1):
            lo, hi = max(start, ci * cr), min(stop, (ci + 1) * cr)
            if hi <= lo:
                continue
            whole = lo == ci * cr and hi == (ci + 1) * cr
            ch = np.zeros(self.chunk, dtype=self.dtype) if whole or not self._chunk_path(ci).exists() \
                else self._read_chunk(ci).copy()
            tail = tuple(slice(0, s) for s in self.shape[1:])
            ch[(slice(lo - ci * cr, hi - ci * cr),) + tail] = data[lo - start: hi - start]
            p = self._chunk_path(ci)
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_bytes(self._encode(ch))

    def resize(self, rows: int) -> None:
        self.meta["shape"][0] = int(rows)
        _write_json(self.path / "zarr.json", self.meta)

    def append(self, data: np.ndarray) -> None:
        data = np.asarray(data).reshape((-1,) + self.shape[1:])
        n = self.shape[0]
        self.resize(n + data.shape[0])
        self.write(n, data)

    def nbytes_on_disk(self) -> int:
        return sum(f.stat().st_size for f in self.path.rglob("*") if f.is_file())


def _level_of(schema: LevelSchema, key: str) -> str | None:
    g = schema.group_of(key)
    return {"atoms": "atom", "edges": "edge", "system": "system"}.get(g)


class AtomicDataZarrWriter:
    def __init__(self, store: str | Path, config: ZarrWriteConfig | None = None) -> None:
        self.root = Path(store)
        self.config = config or ZarrWriteConfig()
        self.schema = LevelSchema()
        if not (self.root / "zarr.json").exists():
            self._init_store()
        self.attrs = json.loads((self.root / "zarr.json").read_text())["attributes"]

    def _init_store(self) -> None:
        _group(self.root, {"num_samples": 0, "fields": {"core": {}, "custom": {}}})
        for g in ("meta", "core", "custom"):
            _group(self.root / g)
        m = self.config.meta
        for name, dt, n in (("atoms_ptr", np.int64, 1), ("edges_ptr", np.int64, 1), ("samples_mask", np.bool_, 0),
                            ("atoms_mask", np.bool_, 0), ("edges_mask", np.bool_, 0)):
            ZarrArray.create(self.root / "meta" / name, (n,), dt, m)

    def _flush_attrs(self) -> None:
        _group(self.root, self.attrs)

    def _cfg(self, key: str) -> ZarrArrayConfig:
        return self.config.field_overrides.get(key, self.config.core)

    def reset(self) -> None:
        import shutil

        if self.root.exists():
            shutil.rmtree(self.root)
        self._init_store()
        self.attrs = json.loads((self.root / "zarr.json").read_text())["attributes"]

    def append(self, batch: Any) -> None:
        """Append every graph of a ``Batch`` (or a list of ``AtomicData``)."""
        from nvalchemi_toolkit_b200.data.batch import Batch

        if not isinstance(batch, Batch):
            batch = Batch.from_data_list(list(batch))
        batch = batch._tight().to("cpu")
        n = batch.num_graphs
        if n == 0:
            return
        meta = {k: ZarrArray(self.root / "meta" / k) for k in ("atoms_ptr", "edges_ptr", "samples_mask", "atoms_mask",
                                                               "edges_mask")}
        a_ptr, e_ptr = meta["atoms_ptr"].read(), meta["edges_ptr"].read()
        a0, e0 = int(a_ptr[-1]), int(e_ptr[-1])
        node_off = batch.batch_ptr.long().numpy()
        fields = self.attrs["fields"]["core"]
        for key, t in batch._storage.items():
            level = _level_of(batch._storage.schema, key)
            if level is None:
                continue
            arr = t.detach().numpy()
            if key == "neighbor_list":  # stored with per-sample local indices
                per_edge = np.repeat(node_off[:-1], batch.num_edges_per_graph.numpy())
                arr = arr - per_edge[:, None]
            if arr.dtype == np.bool_ or arr.dtype.name in _NAMES:
                pass
            else:
                arr = arr.astype(np.float32)
            path = self.root / "core" / key
            if not (path / "zarr.json").exists():
                pre = {"atom": a0, "edge": e0, "system": self.attrs["num_samples"]}[level]
                za = ZarrArray.create(path, (pre,) + arr.shape[1:], arr.dtype, self._cfg(key))
                fields[key] = level
            else:
                za = ZarrArray(path)
            za.append(arr)
        meta["atoms_ptr"].append(a0 + node_off[1:])
        meta["edges_ptr"].append(e0 + batch.edge_ptr.long().numpy()[1:])
        meta["samples_mask"].append(np.ones(n, dtype=np.bool_))
        meta["atoms_mask"].append(np.ones(batch.num_nodes, dtype=np.bool_))
        meta["edges_mask"].append(np.ones(batch.num_edges, dtype=np.bool_))
        self.attrs["num_samples"] += n
        self._flush_attrs()

    write = append

    def add_custom(self, key: str, values: torch.Tensor | np.ndarray, level: str = "system") -> None:
        arr = values.detach().cpu().numpy() if isinstance(values, torch.Tensor) else np.asarray(values)
        za = ZarrArray.create(self.root / "custom" / key, arr.shape, arr.dtype, self.config.custom)
        za.write(0, arr)
        self.attrs["fields"]["custom"][key] = level
        self._flush_attrs()

    def delete(self, indices: Sequence[int]) -> None:
        """Soft delete: clears the sample / atom / edge masks; data stays until :meth:`defragment`."""
        sm, am, em = (ZarrArray(self.root / "meta" / k) for k in ("samples_mask", "atoms_mask", "edges_mask"))
        a_ptr, e_ptr = ZarrArray(self.root / "meta" / "atoms_ptr").read(), ZarrArray(self.root / "meta" / "edges_ptr").read()
        s, a, e = sm.read().copy(), am.read().copy(), em.read().copy()
        for i in indices:
            s[i] = False
            a[a_ptr[i]: a_ptr[i + 1]] = False
            e[e_ptr[i]: e_ptr[i + 1]] = False
        sm.write(0, s)
        am.write(0, a)
        em.write(0, e)

    def defragment(self) -> None:
        """Rewrite the store without soft-deleted samples."""
        reader = AtomicDataZarrReader(self.root)
        keep = [i for i in range(reader.num_total) if reader.samples_mask[i]]
        dicts = [reader.read_raw(i) for i in keep]
        levels = dict(reader.field_levels)
        self.reset()
        from nvalchemi_toolkit_b200.data.batch import Batch

        for lo in range(0, len(dicts), 4096):
            self.append(Batch.from_raw_dicts(dicts[lo: lo + 4096], field_levels={k: {"atom": "node"}.get(v, v)
                                                                                  for k, v in levels.items()}))


class AtomicDataZarrReader:
    """Random access to samples; ``read(i)`` returns ``(dict of tensors, metadata)``."""

    def __init__(self, store: str | Path, device: str | torch.device = "cpu") -> None:
        self.root = Path(store)
        self.device = torch.device(device)
        self.refresh()

    def refresh(self) -> None:
        self.attrs = json.loads((self.root / "zarr.json").read_text())["attributes"]
        self.atoms_ptr = ZarrArray(self.root / "meta" / "atoms_ptr").read()
        self.edges_ptr = ZarrArray(self.root / "meta" / "edges_ptr").read()
        self.samples_mask = ZarrArray(self.root / "meta" / "samples_mask").read()
        self.num_total = int(self.attrs["num_samples"])
        self._live = np.nonzero(self.samples_mask)[0]
        self._arrays = {k: ZarrArray(self.root / "core" / k) for k in self.attrs["fields"]["core"]}
        self._custom = {k: ZarrArray(self.root / "custom" / k) for k in self.attrs["fields"].get("custom", {})}

    @property
    def field_levels(self) -> dict[str, str]:
        return {k: {"atom": "node"}.get(v, v) for k, v in self.attrs["fields"]["core"].items()}

    def __len__(self) -> int:
        return int(self._live.size)

    def get_metadata(self, idx: int) -> tuple[int, int]:
        i = int(self._live[idx])
        return int(self.atoms_ptr[i + 1] - self.atoms_ptr[i]), int(self.edges_ptr[i + 1] - self.edges_ptr[i])

    def read_raw(self, i: int) -> dict[str, torch.Tensor]:
        out = {}
        for key, za in self._arrays.items():
            level = self.attrs["fields"]["core"][key]
            if level == "atom":
                lo, hi = int(self.atoms_ptr[i]), int(self.atoms_ptr[i + 1])
            elif level == "edge":
                lo, hi = int(self.edges_ptr[i]), int(self.edges_ptr[i + 1])
            else:
                lo, hi = i, i + 1
            out[key] = torch.from_numpy(za.read(lo, hi).copy()).to(self.device)
        return out

    def read(self, idx: int) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
        i = int(self._live[idx])
        d = self.read_raw(i)
        return d, {"index": i, "num_atoms": int(d["positions"].shape[0]),
                   "num_edges": int(d["neighbor_list"].shape[0]) if "neighbor_list" in d else 0}

    def read_many(self, indices: Sequence[int]) -> list[tuple[dict[str, torch.Tensor], dict[str, Any]]]:
        """Coalesced read: one span per field covering the requested (sorted) samples, then split."""
        if len(indices) == 0:
            return []
        phys = [int(self._live[i]) for i in indices]
        lo_s, hi_s = min(phys), max(phys) + 1
        spans = {}
        for key, za in self._arrays.items():
            level = self.attrs["fields"]["core"][key]
            ptr = self.atoms_ptr if level == "atom" else self.edges_ptr if level == "edge" else None
            lo, hi = (int(ptr[lo_s]), int(ptr[hi_s])) if ptr is not None else (lo_s, hi_s)
            spans[key] = (za.read(lo, hi), lo, ptr)
        out = []
        for i in phys:
            d = {}
            for key, (arr, lo, ptr) in spans.items():
                a, b = (int(ptr[i]) - lo, int(ptr[i + 1]) - lo) if ptr is not None else (i - lo, i + 1 - lo)
                d[key] = torch.from_numpy(arr[a:b].copy()).to(self.device)
            out.append((d, {"index": i, "num_atoms": int(d["positions"].shape[0]),
                            "num_edges": int(d["neighbor_list"].shape[0]) if "neighbor_list" in d else 0}))
        return out

    def read_custom(self, key: str) -> torch.Tensor:
        return torch.from_numpy(self._custom[key].read().copy())

    def nbytes_on_disk(self) -> int:
        return sum(f.stat().st_size for f in self.root.rglob("*") if f.is_file())
