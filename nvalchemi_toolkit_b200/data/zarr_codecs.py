# SPDX-License-Identifier: Apache-2.0
"""Zarr v3 codec pipeline without the ``zarr`` / ``numcodecs`` packages: ``bytes``, ``gzip``, ``zstd``, ``crc32c``, ``blosc``
(read) and ``sharding_indexed`` (read and write).

The reference writes its stores through zarr-python with per-group ``ZarrArrayConfig(compressors, chunk_size, shard_size)``
(``nvalchemi/data/datapipes/backends/zarr.py:56-183``): Zstd or Blosc(LZ4) compressors and, with ``shard_size``, the
sharding codec that packs many inner chunks plus an offset index into one file.  This module decodes those layouts from
the published Zarr v3 specification.  Compression back ends: ``zstandard`` when importable, else the Zstandard and raw
LZ4 block codecs that ship inside ``pyarrow``; ``zlib`` from the standard library.
"""
from __future__ import annotations

import struct
import zlib
from typing import Any, Sequence

import numpy as np

MAX_U64 = 2 ** 64 - 1


# ---- leaf compressors -----------------------------------------------------------------------------------------------
def _pa_codec(name: str) -> Any:
    import pyarrow as pa

    return pa.Codec(name)


def zstd_compress(raw: bytes, level: int = 3) -> bytes:
    try:
        import zstandard

        return zstandard.ZstdCompressor(level=level).compress(raw)
    except ImportError:
        import pyarrow as pa

        return pa.Codec("zstd", compression_level=level).compress(raw, asbytes=True)


def zstd_decompress(raw: bytes, size: int) -> bytes:
    try:
        import zstandard

        return zstandard.ZstdDecompressor().decompress(raw, max_output_size=max(size, 1))
    except ImportError:
        return _pa_codec("zstd").decompress(raw, decompressed_size=size, asbytes=True)


def zstd_available() -> bool:
    try:
        import zstandard  # noqa: F401

        return True
    except ImportError:
        try:
            _pa_codec("zstd")
            return True
        except Exception:
            return False


_CRC_TABLE: list[int] | None = None


def crc32c(data: bytes) -> int:
    """CRC-32C (Castagnoli), table driven; used for the small shard indices (payload checksums are not re-verified)."""
    global _CRC_TABLE
    if _CRC_TABLE is None:
        table = []
        for i in range(256):
            c = i
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
            table.append(c)
        _CRC_TABLE = table
    crc = 0xFFFFFFFF
    for b in data:
        crc = _CRC_TABLE[(crc ^ b) & 0xFF] ^ (crc >> 8)
    return crc ^ 0xFFFFFFFF


def blosc_decompress(buf: bytes) -> bytes:
    """Decode one Blosc (v1 container) frame: header, block offsets, per-block streams, byte un-shuffle.

    Supported inner compressors: LZ4 / LZ4HC (raw blocks), Zstandard, zlib; filters: none and byte shuffle.  Bit shuffle and
    the BloscLZ compressor raise ``NotImplementedError``."""
    if len(buf) < 16:
        raise ValueError("blosc frame shorter than its header")
    _ver, _verlz, flags, typesize = buf[0], buf[1], buf[2], buf[3]
    nbytes, blocksize, cbytes = struct.unpack_from("<III", buf, 4)
    if cbytes > len(buf):
        raise ValueError("truncated blosc frame")
    if flags & 0x2:  # stored uncompressed
        return bytes(buf[16: 16 + nbytes])
    if flags & 0x4:
        raise NotImplementedError("blosc bit-shuffle is not supported by this reader; use shuffle or noshuffle")
    comp = (flags >> 5) & 0x7
    if comp not in (1, 3, 4):
        raise NotImplementedError(f"blosc inner compressor code {comp} is not supported (lz4, zlib and zstd are)")
    dont_split = bool(flags & 0x10)
    nblocks = (nbytes + blocksize - 1) // blocksize if blocksize else 0
    bstarts = struct.unpack_from(f"<{nblocks}i", buf, 16)
    out = bytearray(nbytes)
    for b in range(nblocks):
        bsize = min(blocksize, nbytes - b * blocksize)
        leftover = bsize != blocksize
        split = (not dont_split) and (not leftover) and typesize > 1 and typesize <= 16 and bsize // typesize >= 128
        nstreams = typesize if split else 1
        neblock = bsize // nstreams
        pos = bstarts[b]
        block = bytearray()
        for _ in range(nstreams):
            (cb,) = struct.unpack_from("<i", buf, pos)
            pos += 4
            chunk = bytes(buf[pos: pos + cb])
            pos += cb
            if cb == neblock:
                block += chunk
            elif comp == 1:
                block += _pa_codec("lz4_raw").decompress(chunk, decompressed_size=neblock, asbytes=True)
            elif comp == 3:
                block += zlib.decompress(chunk)
            else:
                block += zstd_decompress(chunk, neblock)
        if (flags & 0x1) and typesize > 1 and bsize >= typesize:
            n_el = bsize // typesize
            body = np.frombuffer(bytes(block[: n_el * typesize]), dtype=np.uint8).reshape(typesize, n_el).T.tobytes()
            block = bytearray(body) + block[n_el * typesize:]
        out[b * blocksize: b * blocksize + bsize] = block
    return bytes(out)


# ---- codec pipeline -------------------------------------------------------------------------------------------------
SUPPORTED = ("bytes", "gzip", "zstd", "crc32c", "blosc", "sharding_indexed", "transpose")


def check_supported(codecs: Sequence[dict]) -> None:
    for c in codecs:
        if c["name"] not in SUPPORTED:
            raise NotImplementedError(f"Zarr codec '{c['name']}' is not supported by this reader")
        if c["name"] == "sharding_indexed":
            check_supported(c["configuration"]["codecs"])
            check_supported(c["configuration"].get("index_codecs", []))


def decode(raw: bytes, codecs: Sequence[dict], dtype: np.dtype, shape: Sequence[int]) -> np.ndarray:
    """Undo a codec list (array->array filters, one array->bytes serializer, bytes->bytes compressors)."""
    names = [c["name"] for c in codecs]
    ser = next(i for i, n in enumerate(names) if n in ("bytes", "sharding_indexed"))
    size = int(np.prod(shape)) * dtype.itemsize
    for c in reversed(list(codecs[ser + 1:])):
        n = c["name"]
        if n == "gzip":
            raw = zlib.decompress(raw, 16 + zlib.MAX_WBITS)
        elif n == "zstd":
            raw = zstd_decompress(raw, size)
        elif n == "crc32c":
            raw = raw[:-4]
        elif n == "blosc":
            raw = blosc_decompress(raw)
    pre_shape = list(shape)
    for c in codecs[:ser]:  # shapes seen by the serializer after the transposes
        if c["name"] == "transpose":
            pre_shape = [pre_shape[a] for a in c["configuration"]["order"]]
    if names[ser] == "sharding_indexed":
        arr = decode_shard(raw, codecs[ser]["configuration"], dtype, pre_shape)
    else:
        endian = codecs[ser].get("configuration", {}).get("endian", "little")
        dt = dtype.newbyteorder("<" if endian == "little" else ">") if dtype.itemsize > 1 else dtype
        arr = np.frombuffer(raw, dtype=dt).reshape(pre_shape).astype(dtype, copy=False)
    for c in reversed(list(codecs[:ser])):
        if c["name"] == "transpose":
            arr = np.transpose(arr, np.argsort(c["configuration"]["order"]))
    return arr


def encode(arr: np.ndarray, codecs: Sequence[dict], dtype: np.dtype) -> bytes:
    names = [c["name"] for c in codecs]
    ser = next(i for i, n in enumerate(names) if n in ("bytes", "sharding_indexed"))
    arr = np.asarray(arr, dtype=dtype)
    for c in codecs[:ser]:
        if c["name"] == "transpose":
            arr = np.transpose(arr, c["configuration"]["order"])
    if names[ser] == "sharding_indexed":
        raw = encode_shard(arr, codecs[ser]["configuration"], dtype)
    else:
        endian = codecs[ser].get("configuration", {}).get("endian", "little")
        order = "<" if endian == "little" else ">"
        raw = np.ascontiguousarray(arr).astype(dtype.newbyteorder(order) if dtype.itemsize > 1 else dtype, copy=False).tobytes()
    for c in codecs[ser + 1:]:
        n, cfg = c["name"], c.get("configuration", {})
        if n == "gzip":
            co = zlib.compressobj(cfg.get("level", 5), zlib.DEFLATED, 16 + zlib.MAX_WBITS)
            raw = co.compress(raw) + co.flush()
        elif n == "zstd":
            raw = zstd_compress(raw, cfg.get("level", 3))
        elif n == "crc32c":
            raw = raw + struct.pack("<I", crc32c(raw))
        elif n == "blosc":
            raise NotImplementedError("writing blosc chunks is not supported; use zstd or gzip")
    return raw


# ---- sharding_indexed -----------------------------------------------------------------------------------------------
def _index_codecs(cfg: dict) -> list[dict]:
    return cfg.get("index_codecs") or [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "crc32c"}]


def _index_nbytes(cfg: dict, grid: Sequence[int]) -> int:
    n = int(np.prod(grid)) * 16
    for c in _index_codecs(cfg):
        if c["name"] == "crc32c":
            n += 4
        elif c["name"] != "bytes":
            raise NotImplementedError("only bytes (+ crc32c) index codecs have a size known in advance")
    return n


def decode_shard(raw: bytes, cfg: dict, dtype: np.dtype, shard_shape: Sequence[int], fill: Any = 0) -> np.ndarray:
    """One shard file -> array of ``shard_shape``: the index (``[grid..., 2]`` uint64 offset / length, all ones = empty
    inner chunk) sits at the end (default) or the start of the file; inner chunks go through their own codec list."""
    inner = [int(s) for s in cfg["chunk_shape"]]
    grid = [(int(s) + c - 1) // c for s, c in zip(shard_shape, inner)]
    n_idx = _index_nbytes(cfg, grid)
    at_end = cfg.get("index_location", "end") == "end"
    idx_raw = raw[-n_idx:] if at_end else raw[:n_idx]
    icodecs = _index_codecs(cfg)
    if icodecs[-1]["name"] == "crc32c":
        body, (want,) = idx_raw[:-4], struct.unpack("<I", idx_raw[-4:])
        if crc32c(body) != want:
            raise ValueError("shard index checksum mismatch (corrupt shard)")
    index = decode(idx_raw, icodecs, np.dtype("uint64"), grid + [2])
    out = np.full(shard_shape, fill, dtype=dtype)
    for pos in np.ndindex(*grid):
        off, nb = int(index[pos + (0,)]), int(index[pos + (1,)])
        if off == MAX_U64 and nb == MAX_U64:
            continue
        chunk = decode(raw[off: off + nb], cfg["codecs"], dtype, inner)
        sl = tuple(slice(p * c, min((p + 1) * c, s)) for p, c, s in zip(pos, inner, shard_shape))
        out[sl] = chunk[tuple(slice(0, s.stop - s.start) for s in sl)]
    return out


def encode_shard(arr: np.ndarray, cfg: dict, dtype: np.dtype) -> bytes:
    inner = [int(s) for s in cfg["chunk_shape"]]
    shape = list(arr.shape)
    grid = [(s + c - 1) // c for s, c in zip(shape, inner)]
    at_end = cfg.get("index_location", "end") == "end"
    index = np.full(grid + [2], MAX_U64, dtype=np.uint64)
    offset = 0 if at_end else _index_nbytes(cfg, grid)
    parts = []
    for pos in np.ndindex(*grid):
        sl = tuple(slice(p * c, min((p + 1) * c, s)) for p, c, s in zip(pos, inner, shape))
        chunk = np.zeros(inner, dtype=dtype)
        chunk[tuple(slice(0, s.stop - s.start) for s in sl)] = arr[sl]
        blob = encode(chunk, cfg["codecs"], dtype)
        index[pos + (0,)], index[pos + (1,)] = offset, len(blob)
        offset += len(blob)
        parts.append(blob)
    idx = encode(index, _index_codecs(cfg), np.dtype("uint64"))
    return b"".join(parts) + idx if at_end else idx + b"".join(parts)
