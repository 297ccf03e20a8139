# SPDX-License-Identifier: Apache-2.0
"""Zarr v3 store layout, append / delete / defragment, coalesced reads, datapipes and the IO CLI."""
import json

import pytest
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.data.datapipes import (Compose, DataLoader, Dataset, InMemoryDataset, MultiDataset,
                                                   MultiDatasetBatchSampler, MultiDatasetSampler)
from nvalchemi_toolkit_b200.data.zarr_store import (AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArray, ZarrArrayConfig,
                                                    ZarrWriteConfig)
from nvalchemi_toolkit_b200.dynamics.sampler import SizeAwareSampler
from nvalchemi_toolkit_b200.dynamics.sinks import ZarrData
from tests.helpers import random_molecule


def _data(n=7):
    return [random_molecule(3 + i, i, n_edges=2 + i, periodic=True) for i in range(n)]


@pytest.mark.parametrize("compressor", [None, "gzip"])
def test_store_layout_and_roundtrip(tmp_path, compressor):
    data = _data()
    cfg = ZarrWriteConfig(core=ZarrArrayConfig(chunk_rows=8, compressor=compressor))
    w = AtomicDataZarrWriter(tmp_path / "s.zarr", cfg)
    w.append(Batch.from_data_list(data[:4]))
    w.append(Batch.from_data_list(data[4:]))
    root = json.loads((tmp_path / "s.zarr" / "zarr.json").read_text())
    assert root["zarr_format"] == 3 and root["attributes"]["num_samples"] == 7
    assert root["attributes"]["fields"]["core"]["positions"] == "atom"
    assert root["attributes"]["fields"]["core"]["cell"] == "system"
    meta = json.loads((tmp_path / "s.zarr" / "core" / "cell" / "zarr.json").read_text())
    assert meta["shape"] == [7, 3, 3] and meta["codecs"][0]["name"] == "bytes"
    assert ZarrArray(tmp_path / "s.zarr" / "meta" / "atoms_ptr").read().tolist()[:3] == [0, 3, 7]
    r = AtomicDataZarrReader(tmp_path / "s.zarr")
    assert len(r) == 7 and r.get_metadata(2) == (5, 4)
    for i in (0, 3, 6):
        d, m = r.read(i)
        assert torch.allclose(d["positions"], data[i].positions) and torch.equal(d["neighbor_list"], data[i].neighbor_list)
        assert d["cell"].shape == (1, 3, 3)
    many = r.read_many([1, 4, 5])
    assert torch.allclose(many[1][0]["positions"], data[4].positions)


def test_delete_defragment_and_custom(tmp_path):
    data = _data()
    w = AtomicDataZarrWriter(tmp_path / "s.zarr")
    w.append(Batch.from_data_list(data))
    w.add_custom("labels", torch.arange(7), level="system")
    w.delete([1, 5])
    r = AtomicDataZarrReader(tmp_path / "s.zarr")
    assert len(r) == 5 and torch.allclose(r.read(1)[0]["positions"], data[2].positions)
    assert r.read_custom("labels").tolist() == list(range(7))
    w.defragment()
    r.refresh()
    assert r.num_total == 5 and torch.allclose(r.read(4)[0]["positions"], data[6].positions)


def test_dataloader_epochs_resume_and_sharding(tmp_path):
    data = _data(10)
    w = AtomicDataZarrWriter(tmp_path / "s.zarr")
    w.append(Batch.from_data_list(data))
    ds = Dataset(AtomicDataZarrReader(tmp_path / "s.zarr"), transform=Compose([lambda d, m: (d, {**m, "seen": True})]))
    item, meta = ds[2]
    assert meta["seen"] and item.num_nodes == 5
    dl = DataLoader(ds, batch_size=4, shuffle=True, seed=3, prefetch_factor=2)
    dl.set_epoch(0)
    sizes0 = [b.num_nodes for b in dl]
    dl.set_epoch(0)
    assert [b.num_nodes for b in dl] == sizes0 and len(dl) == 3
    dl.set_epoch(1)
    dl.set_epoch(0)
    dl.set_epoch_step(2)
    assert [b.num_nodes for b in dl] == sizes0[2:]
    a, b = DataLoader(ds, batch_size=2), DataLoader(ds, batch_size=2)
    a.set_distributed(0, 2)
    b.set_distributed(1, 2)
    assert sum(x.num_graphs for x in a) == sum(x.num_graphs for x in b) == 5
    raw = DataLoader(Dataset(AtomicDataZarrReader(tmp_path / "s.zarr"), raw=True), batch_size=5)
    first = next(iter(raw))
    assert first.num_graphs == 5 and first.cell.shape == (5, 3, 3)


def test_multidataset_sampler_and_inflight_sampler():
    a, b = InMemoryDataset(_data(4)), InMemoryDataset(_data(6))
    multi = MultiDataset([a, b], weights=[1.0, 3.0])
    assert len(multi) == 10 and multi[5][1]["dataset"] == 1
    s = MultiDatasetSampler(multi, num_samples=400, seed=1)
    idx = list(s)
    frac_b = sum(1 for i in idx if i >= 4) / len(idx)
    assert 0.6 < frac_b < 0.9
    bs = MultiDatasetBatchSampler(MultiDatasetSampler(multi, num_samples=10, rank=0, world_size=2), batch_size=2)
    assert len(list(bs)) == len(bs) == 3
    dl = DataLoader(multi, batch_sampler=bs)
    assert sum(x.num_graphs for x in dl) == 5
    sampler = SizeAwareSampler(a, max_atoms=12, max_batch_size=3)
    assert sampler.build_initial_batch().num_nodes <= 12


def test_zarr_sink_and_cli(tmp_path):
    sink = ZarrData(tmp_path / "sink.zarr")
    batch = Batch.from_data_list(_data(3))
    sink.write(batch, mask=torch.tensor([True, False, True]))
    assert len(sink) == 2 and sink.read().num_graphs == 2
    from nvalchemi_toolkit_b200.data import io_test

    res = io_test.main(["roundtrip", "--samples", "400", "--store", str(tmp_path), "--compressor", "gzip", "--chunk-rows", "4096"])
    assert res["roundtrip_ok"] and res["compression_ratio"] > 1.0
    res2 = io_test.main(["read", res["store"]])
    assert res2["samples"] == 400


def test_sharded_and_compressed_arrays_round_trip(tmp_path):
    """``sharding_indexed`` (index at the end, crc32c-protected) around zstd / gzip inner chunks; partial last shard,
    in-place row updates, and the file count a shard saves."""
    import json

    import numpy as np

    from nvalchemi_toolkit_b200.data import zarr_codecs
    from nvalchemi_toolkit_b200.data.zarr_store import ZarrArray, ZarrArrayConfig

    rng = np.random.default_rng(0)
    data = rng.standard_normal((1000, 3)).astype(np.float32)
    for comp in (None, "gzip", "zstd"):
        a = ZarrArray.create(tmp_path / f"sh_{comp}", data.shape, np.float32,
                             ZarrArrayConfig(chunk_rows=64, shard_rows=256, compressor=comp))
        a.write(0, data)
        assert np.array_equal(ZarrArray(tmp_path / f"sh_{comp}").read(), data)
        assert np.array_equal(a.read(100, 700), data[100:700])
        patch = rng.standard_normal((50, 3)).astype(np.float32)
        a.write(230, patch)  # straddles two shards
        data2 = data.copy()
        data2[230:280] = patch
        assert np.array_equal(a.read(), data2)
        files = [f for f in (tmp_path / f"sh_{comp}").rglob("*") if f.is_file() and f.name != "zarr.json"]
        assert len(files) == 4  # 1000 rows / 256 per shard, instead of 16 chunk files
        meta = json.loads((tmp_path / f"sh_{comp}" / "zarr.json").read_text())
        assert meta["codecs"][0]["name"] == "sharding_indexed" and meta["chunk_grid"]["configuration"]["chunk_shape"] == [256, 3]
    # the index of a shard written by hand per the specification: offsets / lengths, all-ones for a missing inner chunk
    cfg = {"chunk_shape": [2, 3], "codecs": [{"name": "bytes", "configuration": {"endian": "little"}}], "index_location": "start"}
    inner = np.arange(6, dtype="<f4").reshape(2, 3)
    idx = np.full((2, 1, 2), zarr_codecs.MAX_U64, dtype="<u8")
    idx[1, 0] = (32 + 4, inner.nbytes)
    body = idx.tobytes()
    raw = body + zarr_codecs.crc32c(body).to_bytes(4, "little") + inner.tobytes()
    out = zarr_codecs.decode_shard(raw, cfg, np.dtype("float32"), [4, 3], fill=7)
    assert np.array_equal(out[2:], inner) and (out[:2] == 7).all()
    assert zarr_codecs.crc32c(b"123456789") == 0xE3069283  # published check value of CRC-32C


def test_blosc_frames_decode(tmp_path):
    """Blosc v1 frames assembled per the container layout (header, block offsets, split streams, byte shuffle) with LZ4 raw
    blocks, Zstandard and stored blocks."""
    import struct

    import numpy as np
    import pyarrow as pa

    from nvalchemi_toolkit_b200.data import zarr_codecs

    x = (np.arange(4096, dtype=np.float32) * 0.5).astype("<f4")
    raw = x.tobytes()
    typesize, blocksize = 4, 8192

    def frame(comp_code, compress, shuffle):
        blocks, nblocks = [], len(raw) // blocksize
        for b in range(nblocks):
            blk = raw[b * blocksize: (b + 1) * blocksize]
            if shuffle:
                blk = np.frombuffer(blk, np.uint8).reshape(-1, typesize).T.tobytes()
            streams = b""
            ne = blocksize // typesize
            for s in range(typesize):  # split: one stream per byte of the type
                part = blk[s * ne: (s + 1) * ne]
                c = compress(part)
                c = part if len(c) >= len(part) else c
                streams += struct.pack("<i", len(c)) + c
            blocks.append(streams)
        header_len = 16 + 4 * nblocks
        starts, pos = [], header_len
        for blk in blocks:
            starts.append(pos)
            pos += len(blk)
        flags = (comp_code << 5) | (1 if shuffle else 0)
        head = bytes([2, 1, flags, typesize]) + struct.pack("<III", len(raw), blocksize, pos)
        return head + struct.pack(f"<{nblocks}i", *starts) + b"".join(blocks)

    lz4 = lambda p: pa.Codec("lz4_raw").compress(p, asbytes=True)  # noqa: E731
    zst = lambda p: zarr_codecs.zstd_compress(p, 3)  # noqa: E731
    for code, fn in ((1, lz4), (4, zst)):
        for shuffle in (False, True):
            assert zarr_codecs.blosc_decompress(frame(code, fn, shuffle)) == raw
    stored = bytes([2, 1, 0x2, typesize]) + struct.pack("<III", len(raw), blocksize, 16 + len(raw)) + raw
    assert zarr_codecs.blosc_decompress(stored) == raw
    codecs = [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "blosc", "configuration": {}}]
    assert np.array_equal(zarr_codecs.decode(frame(1, lz4, True), codecs, np.dtype("float32"), [4096]), x)


def test_io_cli_sweep_edges_shards_and_read_orders(tmp_path, capsys):
    """The IO benchmark command: two dataset sizes, edge arrays with their own shard size, every read mode and order; the
    block shuffle keeps samples of a block together; options without a command mean ``roundtrip``."""
    from nvalchemi_toolkit_b200.data import io_test

    res = io_test.main(["-n", "60", "-n", "90", "--edges-per-atom", "4", "--compressor", "zstd", "--chunk-size", "512",
                        "--shard-size", "2048", "--edge-shard-size", "4096", "--read-mode", "both", "--read-order", "all",
                        "--read-block-size", "16", "--output-dir", str(tmp_path)])
    assert [r["samples"] for r in res] == [60, 90]
    for r in res:
        assert r["roundtrip_ok"] and r["edges"] == 4 * r["atoms"] and r["compression_ratio"] > 1.0
        assert {(p["mode"], p["order"]) for p in r["reads"]} == {(m, o) for m in io_test.READ_MODES for o in io_test.READ_ORDERS}
        assert all(p["samples"] == r["samples"] and p["atoms"] == r["atoms"] for p in r["reads"])
        assert abs(r["estimated_raw_bytes"] - r["raw_bytes"]) < 0.15 * r["raw_bytes"]
    out = capsys.readouterr().out
    assert "edge-shard=4096" in out and "block-shuffle" in out
    idx = io_test.read_indices(50, "block-shuffle", seed=3, block=8)
    assert sorted(idx) == list(range(50)) and idx != list(range(50))
    assert all(idx[k + 1] == idx[k] + 1 for k in range(len(idx) - 1) if (idx[k] + 1) % 8 and idx[k] + 1 < 50)
    assert io_test.fmt_bytes(1536) == "1.5 KiB" and io_test.fmt_bytes(12) == "12 B"


def test_decoded_chunk_cache_sees_rewrites(tmp_path):
    """Repeated reads of one chunk decode it once; a rewrite by ANOTHER array object is picked up (size / mtime stamp)."""
    import numpy as np

    from nvalchemi_toolkit_b200.data.zarr_store import ZarrArray, ZarrArrayConfig

    a = ZarrArray.create(tmp_path / "x", (0, 3), np.float32, ZarrArrayConfig(chunk_rows=8, compressor="gzip"))
    a.append(np.arange(48, dtype=np.float32).reshape(16, 3))
    calls = []
    orig = a._decode
    a._decode = lambda raw: (calls.append(1), orig(raw))[1]
    first = a.read(2, 5)
    assert np.array_equal(a.read(2, 5), first) and len(calls) == 1
    first[0, 0] = -1.0  # the caller owns what read() returns
    assert a.read(2, 3)[0, 0] == 6.0
    b = ZarrArray(tmp_path / "x")
    b.write(2, np.full((1, 3), 99.0, dtype=np.float32))
    import os
    import time

    os.utime(b._chunk_path(0), ns=(time.time_ns(), time.time_ns() + 1_000_000))
    assert a.read(2, 3)[0, 0] == 99.0 and len(calls) == 2


def test_multidataset_sampler_counts_epochs_sharding_and_homogeneous_batches():
    from nvalchemi_toolkit_b200.data.datapipes import counts_from_weights

    assert counts_from_weights([1, 1, 1], 10) == [4, 3, 3] and counts_from_weights([3, 1], 8) == [6, 2]
    with pytest.raises(ValueError):
        counts_from_weights([0, 0], 5)
    a = InMemoryDataset(_data(6))
    b = InMemoryDataset(_data(3))
    multi = MultiDataset([a, b])
    # proportional by length, without replacement: one epoch of len(multi) samples is a permutation of everything
    s = MultiDatasetSampler(multi, replacement=False, seed=3)
    assert sorted(s) == list(range(9))
    first = list(s)
    s.set_epoch(1)
    assert list(s) != first and sorted(s) == list(range(9))
    # explicit rates: exact counts; the small dataset wraps around only after every sample was seen
    s = MultiDatasetSampler(multi, num_samples=12, weights=[1, 1], replacement=False, seed=0)
    idx = list(s)
    from_b = [i for i in idx if i >= 6]
    assert len(idx) == 12 and len(from_b) == 6 and sorted(from_b) == [6, 6, 7, 7, 8, 8]
    assert list(MultiDatasetSampler(multi, shuffle=False, replacement=False)) == list(range(9))
    # ranks draw equally many samples; together they cover the epoch order (padded by its head)
    shards = [list(MultiDatasetSampler(multi, num_samples=10, seed=5, rank=r, world_size=4)) for r in range(4)]
    order = MultiDatasetSampler(multi, num_samples=10, seed=5).epoch_order()
    assert [len(x) for x in shards] == [3, 3, 3, 3]
    merged = [shards[i % 4][i // 4] for i in range(12)]
    assert merged[:10] == order and merged[10:] == order[:2]
    assert [len(list(MultiDatasetSampler(multi, num_samples=10, rank=r, world_size=4, drop_last=True))) for r in range(4)] == [2] * 4
    # every batch inside one dataset
    bs = MultiDatasetBatchSampler(MultiDatasetSampler(multi, num_samples=18, weights=[2, 1], seed=2), batch_size=4, homogeneous=True)
    batches = list(bs)
    assert sum(len(x) for x in batches) == 18 and len(bs) == len(batches)
    assert all(len({multi.locate(i)[0] for i in x}) == 1 for x in batches)
    with pytest.raises(ValueError, match="empty dataset"):
        MultiDatasetSampler(MultiDataset([a, InMemoryDataset([])]), weights=[1, 1])


def test_fixed_composition_batches_policies_and_sharding():
    from nvalchemi_toolkit_b200.data.datapipes import FixedCompositionBatchSampler, num_batches_from_policy

    big, small = InMemoryDataset(_data(12)), InMemoryDataset(_data(4))
    multi = MultiDataset([big, small])
    s = FixedCompositionBatchSampler(multi, batch_size=8, weights=[3, 1], replacement=False, seed=1)
    assert s.samples_per_dataset == [6, 2] and s.num_batches == 2 and len(s) == 2
    batches = list(s)
    for b in batches:
        assert sum(i < 12 for i in b) == 6 and sum(i >= 12 for i in b) == 2    # the same composition in every batch
    flat = [i for b in batches for i in b]
    assert len(set(flat)) == len(flat) == 16                                    # no repeats inside the epoch
    s.set_epoch(1)
    assert list(s) != batches
    # policies: until the first / last dataset has been seen once
    assert num_batches_from_policy("min_size", [12, 4], [4, 4], 8, True) == 1
    assert num_batches_from_policy("max_size", [12, 4], [4, 4], 8, True) == 3
    assert num_batches_from_policy("dataset_size", [12, 4], [4, 4], 8, True) == 2
    with pytest.raises(ValueError, match="replacement"):
        num_batches_from_policy("max_size", [12, 4], [4, 4], 8, False)
    bal = FixedCompositionBatchSampler.balanced(multi, 8, epoch_policy="max_size", seed=0)
    assert bal.samples_per_dataset == [4, 4] and bal.num_batches == 3
    small_seen = [i for b in bal.epoch_batches() for i in b if i >= 12]
    assert len(small_seen) == 12 and set(small_seen) == {12, 13, 14, 15}         # the small set wrapped around three times
    assert small_seen[:4] != small_seen[4:8] or small_seen[4:8] != small_seen[8:]  # ... through fresh permutations
    # two ranks: strided shares of the same epoch; three batches are padded to four unless drop_last
    r0 = FixedCompositionBatchSampler.balanced(multi, 8, epoch_policy="max_size", rank=0, world_size=2)
    r1 = FixedCompositionBatchSampler.balanced(multi, 8, epoch_policy="max_size", rank=1, world_size=2)
    assert len(r0) == len(r1) == 2 and list(r0)[0] == bal.epoch_batches()[0] and list(r1)[1] == bal.epoch_batches()[0]
    d0 = FixedCompositionBatchSampler.balanced(multi, 8, epoch_policy="max_size", rank=0, world_size=2, drop_last=True)
    assert len(d0) == 1 and len(list(d0)) == 1
    with pytest.raises(ValueError, match="smaller than its share"):
        FixedCompositionBatchSampler(multi, 16, weights=[1, 1], replacement=False)
    # through the loader: batches arrive with the composition intact
    loader = DataLoader(multi, batch_sampler=FixedCompositionBatchSampler(multi, 8, weights=[3, 1], replacement=False))
    assert [b.num_graphs for b in loader] == [8, 8]


def test_dataset_field_names_get_batch_and_close(tmp_path):
    w = AtomicDataZarrWriter(tmp_path / "s.zarr")
    data = _data(5)
    w.write(data)
    with Dataset(AtomicDataZarrReader(tmp_path / "s.zarr")) as ds:
        assert {"positions", "atomic_numbers"} <= set(ds.field_names)
        b = ds.get_batch([3, 0])
        assert b.num_graphs == 2 and torch.allclose(b[0].positions, data[3].positions)
    with pytest.raises(RuntimeError):
        ds.fetch([0])  # the worker pool is gone after close


def test_crc32c_known_vectors_and_codec_checks():
    """Castagnoli CRC against the published check values (RFC 3720 appendix B.4) and the codec-chain validation."""
    import numpy as np

    from nvalchemi_toolkit_b200.data import zarr_codecs

    assert zarr_codecs.crc32c(b"") == 0
    assert zarr_codecs.crc32c(b"123456789") == 0xE3069283
    assert zarr_codecs.crc32c(bytes(32)) == 0x8A9136AA
    assert zarr_codecs.crc32c(bytes([0xFF] * 32)) == 0x62A8AB43
    assert zarr_codecs.crc32c(bytes(range(32))) == 0x46DD794E
    with pytest.raises((ValueError, NotImplementedError)):
        zarr_codecs.check_supported([{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "lz77-homebrew"}])
    chain = [{"name": "bytes", "configuration": {"endian": "little"}}, {"name": "gzip", "configuration": {"level": 1}}]
    arr = np.arange(24, dtype="<f4").reshape(4, 6)
    raw = zarr_codecs.encode(arr, chain, np.dtype("float32"))
    assert np.array_equal(zarr_codecs.decode(raw, chain, np.dtype("float32"), [4, 6]), arr)
    big = [{"name": "bytes", "configuration": {"endian": "big"}}]
    assert zarr_codecs.encode(arr, big, np.dtype("float32")) == arr.astype(">f4").tobytes()
    assert np.array_equal(zarr_codecs.decode(arr.astype(">f4").tobytes(), big, np.dtype("float32"), [4, 6]), arr)
