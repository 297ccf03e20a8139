# SPDX-License-Identifier: Apache-2.0
"""Datapipes: readers, datasets with prefetch, a batching dataloader, multi-dataset sampling, transforms.

Reference: ``nvalchemi/data/datapipes/{backends/base,dataset,dataloader,multidataset,in_memory_dataset,samplers}.py`` and
``data/transforms/compose.py``.  A ``Reader`` returns raw dictionaries of tensors plus metadata; ``Dataset`` turns them
into ``AtomicData`` (or keeps them raw for ``Batch.from_raw_dicts``), prefetching with a thread pool and, on CUDA, a side
stream; ``DataLoader`` assembles ``Batch`` objects, reads several batches per window (``prefetch_factor``), supports
``set_epoch`` (shuffle seed), ``set_epoch_step`` (mid-epoch resume) and ``set_distributed`` (rank sharding)."""
from __future__ import annotations

import abc
import concurrent.futures as cf
import math
from typing import Any, Callable, Iterator, Protocol, Sequence

import torch

from nvalchemi_toolkit_b200.data.atomic_data import AtomicData
from nvalchemi_toolkit_b200.data.batch import Batch


class Reader(abc.ABC):
    """Random-access source of samples."""

    @abc.abstractmethod
    def __len__(self) -> int: ...

    @abc.abstractmethod
    def read(self, idx: int) -> tuple[dict[str, torch.Tensor], dict[str, Any]]: ...

    def read_many(self, indices: Sequence[int]) -> list[tuple[dict[str, torch.Tensor], dict[str, Any]]]:
        return [self.read(i) for i in indices]

    @property
    def field_levels(self) -> dict[str, str]:
        return {}

    def get_metadata(self, idx: int) -> tuple[int, int]:
        d, m = self.read(idx)
        return int(d["positions"].shape[0]), int(m.get("num_edges", 0))


from nvalchemi_toolkit_b200.data.transforms import Compose  # noqa: E402,F401  (kept importable from here)


def _to_atomic_data(d: dict[str, torch.Tensor], levels: dict[str, str]) -> AtomicData:
    known = {k: v for k, v in d.items() if k in AtomicData.model_fields}
    data = AtomicData(**known)
    for k, v in d.items():
        if k in known:
            continue
        lvl = levels.get(k, "node")
        {"node": data.add_node_property, "edge": data.add_edge_property, "system": data.add_system_property}[lvl](k, v)
    return data


class BatchDatasetProtocol(Protocol):
    """What :class:`DataLoader` and the samplers need from a dataset (reference ``datapipes/dataset.py:78-142``):
    a length, indexed samples ``(item, metadata)``, ``get_metadata(i) -> (num_atoms, num_edges)`` for size-aware
    sampling and, optionally, ``fetch(indices) -> Future[list[(item, metadata)]]`` for windowed asynchronous reads."""

    def __len__(self) -> int: ...

    def __getitem__(self, idx: int) -> tuple[Any, dict[str, Any]]: ...

    def get_metadata(self, idx: int) -> tuple[int, int]: ...


class DistributedSamplerProtocol(Protocol):
    """A sampler that hands each rank its share of an epoch (``torch.utils.data.DistributedSampler`` satisfies it, and so
    do the multi-dataset samplers below): ``num_replicas``, ``rank``, ``set_epoch(epoch)``, iteration over indices."""

    num_replicas: int
    rank: int

    def set_epoch(self, epoch: int) -> None: ...

    def __iter__(self) -> Iterator[int]: ...

    def __len__(self) -> int: ...


class Dataset:
    """Samples as ``(AtomicData, metadata)``; implements the sampler protocol (``get_metadata``)."""

    def __init__(self, reader: Reader, transform: Callable | None = None, device: str | torch.device = "cpu",
                 num_workers: int = 2, raw: bool = False) -> None:
        self.reader, self.transform, self.device, self.raw = reader, transform, torch.device(device), raw
        self._pool = cf.ThreadPoolExecutor(max_workers=max(1, num_workers))
        self._stream = torch.cuda.Stream() if self.device.type == "cuda" else None

    def __len__(self) -> int:
        return len(self.reader)

    def get_metadata(self, idx: int) -> tuple[int, int]:
        return self.reader.get_metadata(idx)

    def _finish(self, d: dict[str, torch.Tensor], meta: dict[str, Any]) -> tuple[Any, dict[str, Any]]:
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                d = {k: v.pin_memory().to(self.device, non_blocking=True) for k, v in d.items()}
            meta = {**meta, "_event": self._stream.record_event()}
        item: Any = d if self.raw else _to_atomic_data(d, self.reader.field_levels)
        if self.transform is not None:
            item, meta = self.transform(item, meta)
        return item, meta

    def __getitem__(self, idx: int) -> tuple[Any, dict[str, Any]]:
        return self._finish(*self.reader.read(idx))

    @property
    def field_names(self) -> list[str]:
        """Names of the tensors a sample carries (from the reader's level table, else from sample 0)."""
        levels = getattr(self.reader, "field_levels", None)
        if levels:
            return sorted(levels)
        return sorted(self.reader.read(0)[0]) if len(self) else []

    def get_batch(self, indices: Sequence[int]) -> Batch:
        """One ``Batch`` from a fused read of ``indices`` (the reader sees them as one window)."""
        items = [self._finish(d, m) for d, m in self.reader.read_many(list(indices))]
        for _, m in items:
            ev = m.get("_event") if isinstance(m, dict) else None
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
        if self.raw:
            return Batch.from_raw_dicts([it for it, _ in items], field_levels=getattr(self.reader, "field_levels", {}))
        return Batch.from_data_list([it for it, _ in items])

    def close(self) -> None:
        """Stop the read workers (pending reads are abandoned) and close the reader."""
        self._pool.shutdown(wait=False, cancel_futures=True)
        close = getattr(self.reader, "close", None)
        if callable(close):
            close()

    def __enter__(self) -> "Dataset":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    def fetch(self, indices: Sequence[int]) -> "cf.Future[list[tuple[Any, dict[str, Any]]]]":
        """Asynchronous fused read of several samples (one reader window)."""
        return self._pool.submit(lambda: [self._finish(d, m) for d, m in self.reader.read_many(list(indices))])


class InMemoryDataset(Dataset):
    """Dataset over a list of ``AtomicData`` kept in memory (optionally resident on the device)."""

    class _ListReader(Reader):
        def __init__(self, items: Sequence[AtomicData]) -> None:
            self.items = list(items)
            # level of every field (custom ones included), so that fused reads rebuild samples with the right levels
            self._levels: dict[str, str] = {}
            for d in self.items:
                for k in d._tensor_items():
                    if k not in self._levels and d.level_of(k) is not None:
                        self._levels[k] = d.level_of(k)

        @property
        def field_levels(self) -> dict[str, str]:
            return self._levels

        def __len__(self) -> int:
            return len(self.items)

        def read(self, idx: int) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
            d = self.items[idx]
            return d._tensor_items(), {"index": idx, "num_atoms": d.num_nodes, "num_edges": d.num_edges}

        def get_metadata(self, idx: int) -> tuple[int, int]:
            return self.items[idx].num_nodes, self.items[idx].num_edges

    def __init__(self, items: Sequence[AtomicData], transform: Callable | None = None,
                 device: str | torch.device = "cpu") -> None:
        items = [d.to(device) for d in items] if torch.device(device).type != "cpu" else list(items)
        super().__init__(self._ListReader(items), transform=transform, device="cpu", num_workers=1)
        self.items = items

    def __getitem__(self, idx: int) -> tuple[Any, dict[str, Any]]:
        item, meta = self.items[idx].clone(), {"index": idx}
        return self.transform(item, meta) if self.transform is not None else (item, meta)

    @classmethod
    def from_dataset(cls, ds: Dataset, device: str | torch.device = "cpu") -> "InMemoryDataset":
        return cls([ds[i][0] for i in range(len(ds))], device=device)


class MultiDataset:
    """Concatenation of datasets with per-dataset sampling weights."""

    def __init__(self, datasets: Sequence[Dataset], weights: Sequence[float] | None = None) -> None:
        self.datasets = list(datasets)
        self.weights = list(weights) if weights is not None else [1.0] * len(self.datasets)
        self.offsets = [0]
        for d in self.datasets:
            self.offsets.append(self.offsets[-1] + len(d))

    def __len__(self) -> int:
        return self.offsets[-1]

    def locate(self, idx: int) -> tuple[int, int]:
        for k in range(len(self.datasets)):
            if idx < self.offsets[k + 1]:
                return k, idx - self.offsets[k]
        raise IndexError(idx)

    def __getitem__(self, idx: int) -> tuple[Any, dict[str, Any]]:
        k, j = self.locate(idx)
        item, meta = self.datasets[k][j]
        return item, {**meta, "dataset": k}

    def get_metadata(self, idx: int) -> tuple[int, int]:
        k, j = self.locate(idx)
        return self.datasets[k].get_metadata(j)


def counts_from_weights(weights: Sequence[float], total: int) -> list[int]:
    """Integer sample counts proportional to ``weights`` that sum to ``total`` exactly (largest-remainder rounding), so an
    epoch draws a deterministic number of samples from every dataset instead of a multinomial one."""
    w = torch.tensor(list(weights), dtype=torch.float64)
    if w.numel() == 0 or bool((w < 0).any()) or float(w.sum()) <= 0:
        raise ValueError("weights must be non-negative with a positive sum")
    exact = w / w.sum() * total
    base = exact.floor().long()
    rest = int(total - int(base.sum()))
    if rest:
        order = torch.argsort(exact - base, descending=True, stable=True)[:rest]
        base[order] += 1
    return base.tolist()


class MultiDatasetSampler:
    """Global indices of a :class:`MultiDataset` at per-dataset rates (reference ``data/datapipes/samplers.py:237-420``).

    ``weights`` (default: the dataset lengths, i.e. proportional sampling) fix how many of the ``num_samples`` indices of an
    epoch come from each dataset (exact counts, not a multinomial draw).  ``replacement=False`` walks a fresh permutation
    of each dataset and wraps around when a dataset is asked for more samples than it has (every sample is seen before any
    repeats); ``shuffle=False`` keeps storage order.  Ranks take strided shares of the same epoch order; ``drop_last``
    trims the order to a multiple of the world size, otherwise it is padded by repeating its head so that every rank
    draws the same number of samples."""

    def __init__(self, multi: MultiDataset, num_samples: int | None = None, seed: int = 0, rank: int = 0,
                 world_size: int = 1, weights: Sequence[float] | None = None, replacement: bool = True, shuffle: bool = True,
                 drop_last: bool = False) -> None:
        self.multi, self.seed, self.rank, self.world_size, self.epoch = multi, seed, rank, world_size, 0
        self.num_samples = num_samples if num_samples is not None else len(multi)
        if self.num_samples < 1:
            raise ValueError(f"num_samples must be >= 1, got {self.num_samples}")
        self.lengths = [len(d) for d in multi.datasets]
        self.weights = list(weights) if weights is not None else (
            list(multi.weights) if any(w != 1.0 for w in multi.weights) else [float(n) for n in self.lengths])
        if len(self.weights) != len(self.lengths):
            raise ValueError("one weight per dataset")
        if any(w > 0 and n == 0 for w, n in zip(self.weights, self.lengths)):
            raise ValueError("an empty dataset cannot have a positive sampling weight")
        self.replacement, self.shuffle, self.drop_last = replacement, shuffle, drop_last

    @property
    def num_replicas(self) -> int:
        return self.world_size

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _per_rank(self) -> int:
        n, w = self.num_samples, self.world_size
        return n // w if self.drop_last else math.ceil(n / w)

    def __len__(self) -> int:
        return self._per_rank()

    def epoch_order(self) -> list[int]:
        """The epoch's global order before sharding (the same on every rank)."""
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        counts = counts_from_weights(self.weights, self.num_samples)
        parts = []
        for k, (cnt, n) in enumerate(zip(counts, self.lengths)):
            if cnt == 0:
                continue
            if self.replacement and self.shuffle:
                local = torch.randint(0, n, (cnt,), generator=g)
            else:
                reps = -(-cnt // n)
                chunks = [torch.randperm(n, generator=g) if self.shuffle else torch.arange(n) for _ in range(reps)]
                local = torch.cat(chunks)[:cnt]
            parts.append(local + self.multi.offsets[k])
        order = torch.cat(parts)
        if self.shuffle:
            order = order[torch.randperm(order.numel(), generator=g)]
        return order.tolist()

    def __iter__(self) -> Iterator[int]:
        order = self.epoch_order()
        per, w = self._per_rank(), self.world_size
        if self.drop_last:
            order = order[: per * w]
        elif len(order) < per * w:
            order = order + order[: per * w - len(order)]
        return iter(order[self.rank:: w])


class MultiDatasetBatchSampler:
    """Batches of indices from a :class:`MultiDatasetSampler`.  ``homogeneous=True`` keeps every batch inside ONE dataset
    (multi-fidelity training where datasets carry different label sets or loss heads): indices are bucketed per dataset in
    the sampler's order and a batch is emitted whenever a bucket fills; the partial buckets follow at the end of the epoch
    unless ``drop_last``."""

    def __init__(self, sampler: MultiDatasetSampler, batch_size: int, drop_last: bool = False, homogeneous: bool = False) -> None:
        self.sampler, self.batch_size, self.drop_last, self.homogeneous = sampler, batch_size, drop_last, homogeneous

    def set_epoch(self, epoch: int) -> None:
        self.sampler.set_epoch(epoch)

    def __iter__(self) -> Iterator[list[int]]:
        if not self.homogeneous:
            buf: list[int] = []
            for i in self.sampler:
                buf.append(i)
                if len(buf) == self.batch_size:
                    yield buf
                    buf = []
            if buf and not self.drop_last:
                yield buf
            return
        buckets: dict[int, list[int]] = {}
        for i in self.sampler:
            k = self.sampler.multi.locate(i)[0]
            b = buckets.setdefault(k, [])
            b.append(i)
            if len(b) == self.batch_size:
                yield b
                buckets[k] = []
        if not self.drop_last:
            for k in sorted(buckets):
                if buckets[k]:
                    yield buckets[k]

    def __len__(self) -> int:
        n = len(self.sampler)
        if not self.homogeneous:
            return n // self.batch_size if self.drop_last else math.ceil(n / self.batch_size)
        return sum(1 for _ in self)  # depends on how the epoch's indices fall into the buckets


def num_batches_from_policy(policy: str, lengths: Sequence[int], per_batch: Sequence[int], batch_size: int, replacement: bool) -> int:
    """Epoch length of a fixed-composition sampler (reference ``samplers.py:196-235``).  ``dataset_size``: as many batches
    as the concatenated data fill (with replacement) or as the first dataset to run out allows (without);
    ``min_size`` / ``max_size``: until the first / the last contributing dataset has been seen once (``max_size`` makes
    the smaller ones repeat, so it needs ``replacement``)."""
    pairs = [(n, c) for n, c in zip(lengths, per_batch) if c > 0]
    if not pairs:
        raise ValueError("at least one dataset must contribute samples to a batch")
    if replacement:
        lo, hi = min(-(-n // c) for n, c in pairs), max(-(-n // c) for n, c in pairs)
    else:
        lo, hi = min(n // c for n, c in pairs), max(n // c for n, c in pairs)
    if policy == "dataset_size":
        return -(-sum(lengths) // batch_size) if replacement else lo
    if policy == "min_size":
        return lo
    if policy == "max_size":
        if not replacement and hi > lo:
            raise ValueError("epoch_policy='max_size' repeats the smaller datasets: it needs replacement=True")
        return hi
    raise ValueError("epoch_policy must be 'dataset_size', 'min_size' or 'max_size'")


class FixedCompositionBatchSampler:
    """Every batch holds the SAME number of samples from each dataset (reference ``samplers.py:423-789``).

    ``weights`` (default: the dataset lengths) are turned into per-batch counts with :func:`counts_from_weights`, so with
    ``weights=[3, 1]`` and ``batch_size=8`` each batch has 6 samples of the first dataset and 2 of the second, whatever
    their sizes: a small high-fidelity set is seen at a fixed rate in every optimiser step instead of in bursts.
    Without ``replacement`` each dataset is walked through a fresh permutation per epoch (no repeats inside an epoch; the
    epoch ends when the policy says so); with it the permutation wraps around.  Ranks take strided shares of the epoch's
    batches; ``drop_last`` trims the number of batches to a multiple of the world size, otherwise the head of the epoch
    is repeated so that every rank runs the same number of steps."""

    def __init__(self, multi: MultiDataset, batch_size: int, weights: Sequence[float] | None = None,
                 num_batches: int | None = None, epoch_policy: str = "dataset_size", replacement: bool = True,
                 shuffle: bool = True, seed: int = 0, rank: int = 0, world_size: int = 1, drop_last: bool = False) -> None:
        self.multi, self.batch_size, self.replacement, self.shuffle = multi, int(batch_size), replacement, shuffle
        self.seed, self.rank, self.world_size, self.drop_last, self.epoch = seed, rank, world_size, drop_last, 0
        self.lengths = [len(d) for d in multi.datasets]
        w = list(weights) if weights is not None else [float(n) for n in self.lengths]
        if len(w) != len(self.lengths):
            raise ValueError("one weight per dataset")
        self.samples_per_dataset = counts_from_weights(w, self.batch_size)
        if any(c > 0 and n == 0 for c, n in zip(self.samples_per_dataset, self.lengths)):
            raise ValueError("an empty dataset cannot contribute to a batch")
        if not replacement and any(c > n for c, n in zip(self.samples_per_dataset, self.lengths)):
            raise ValueError("a dataset is smaller than its share of one batch: use replacement=True")
        self.num_batches = int(num_batches) if num_batches is not None else num_batches_from_policy(
            epoch_policy, self.lengths, self.samples_per_dataset, self.batch_size, replacement)
        if self.num_batches < 1:
            raise ValueError("the epoch would hold no batch")
        if not replacement:
            most = min(n // c for n, c in zip(self.lengths, self.samples_per_dataset) if c > 0)
            if self.num_batches > most:
                raise ValueError(f"{self.num_batches} batches without replacement need more samples than the smallest "
                                 f"contributing dataset holds ({most} batches at most)")

    @classmethod
    def balanced(cls, multi: MultiDataset, batch_size: int, **kwargs: Any) -> "FixedCompositionBatchSampler":
        """Equal shares of every batch for all datasets."""
        return cls(multi, batch_size, weights=[1.0] * len(multi.datasets), **kwargs)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _per_rank(self) -> int:
        return self.num_batches // self.world_size if self.drop_last else -(-self.num_batches // self.world_size)

    def __len__(self) -> int:
        return self._per_rank()

    def epoch_batches(self) -> list[list[int]]:
        """All batches of the epoch before sharding (the same on every rank)."""
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        streams = []
        for n, c in zip(self.lengths, self.samples_per_dataset):
            need = c * self.num_batches
            if need == 0:
                streams.append(None)
                continue
            reps = -(-need // n)
            streams.append(torch.cat([torch.randperm(n, generator=g) if self.shuffle else torch.arange(n) for _ in range(reps)])[:need])
        out = []
        for b in range(self.num_batches):
            parts = [st[b * c: (b + 1) * c] + off for st, c, off in zip(streams, self.samples_per_dataset, self.multi.offsets)
                     if st is not None]
            batch = torch.cat(parts)
            if self.shuffle:
                batch = batch[torch.randperm(batch.numel(), generator=g)]
            out.append(batch.tolist())
        return out

    def __iter__(self) -> Iterator[list[int]]:
        batches = self.epoch_batches()
        per, w = self._per_rank(), self.world_size
        if self.drop_last:
            batches = batches[: per * w]
        elif len(batches) < per * w:
            batches = batches + batches[: per * w - len(batches)]
        return iter(batches[self.rank:: w])


class DataLoader:
    """Yields ``Batch`` objects; reads ``prefetch_factor`` batches per window ahead of consumption."""

    def __init__(self, dataset: Any, batch_size: int = 1, shuffle: bool = False, drop_last: bool = False,
                 prefetch_factor: int = 2, seed: int = 0, batch_sampler: Any = None,
                 device: str | torch.device | None = None) -> None:
        self.dataset, self.batch_size, self.shuffle, self.drop_last = dataset, batch_size, shuffle, drop_last
        self.prefetch_factor, self.seed, self.batch_sampler = max(1, prefetch_factor), seed, batch_sampler
        self.device = torch.device(device) if device is not None else None
        self.epoch, self.start_step = 0, 0
        self.rank, self.world_size = 0, 1

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch
        if self.batch_sampler is not None and hasattr(self.batch_sampler, "set_epoch"):
            self.batch_sampler.set_epoch(epoch)

    def set_epoch_step(self, step: int) -> None:
        """Skip the first ``step`` batches of the next iteration (resume in the middle of an epoch)."""
        self.start_step = int(step)

    def set_distributed(self, rank: int, world_size: int) -> None:
        self.rank, self.world_size = rank, world_size

    def _batches(self) -> list[list[int]]:
        if self.batch_sampler is not None:
            return list(self.batch_sampler)
        n = len(self.dataset)
        order = torch.randperm(n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist() \
            if self.shuffle else list(range(n))
        if self.world_size > 1:
            per = math.ceil(n / self.world_size)
            order = (order + order[: per * self.world_size - n])[self.rank:: self.world_size]
        out = [order[i: i + self.batch_size] for i in range(0, len(order), self.batch_size)]
        if self.drop_last and out and len(out[-1]) < self.batch_size:
            out.pop()
        return out

    def __len__(self) -> int:
        return len(self._batches())

    def _collate(self, items: list[tuple[Any, dict[str, Any]]]) -> Batch:
        for _, m in items:
            ev = m.get("_event") if isinstance(m, dict) else None
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)
        first = items[0][0]
        if isinstance(first, dict):
            levels = getattr(getattr(self.dataset, "reader", None), "field_levels", {})
            b = Batch.from_raw_dicts([it for it, _ in items], field_levels=levels)
        else:
            b = Batch.from_data_list([it for it, _ in items])
        return b.to(self.device, non_blocking=True) if self.device is not None else b

    def __iter__(self) -> Iterator[Batch]:
        batches = self._batches()[self.start_step:]
        self.start_step = 0
        fetch = getattr(self.dataset, "fetch", None)
        if fetch is None:
            for idx in batches:
                yield self._collate([self.dataset[i] for i in idx])
            return
        pending: list[Any] = []
        it = iter(batches)

        def submit() -> None:
            window = [b for b in (next(it, None) for _ in range(self.prefetch_factor)) if b is not None]
            if window:
                flat = [i for b in window for i in b]
                pending.append((window, fetch(flat)))

        submit()
        while pending:
            window, fut = pending.pop(0)
            submit()  # the next window is read while this one is consumed
            items = fut.result()
            pos = 0
            for b in window:
                yield self._collate(items[pos: pos + len(b)])
                pos += len(b)


from nvalchemi_toolkit_b200.data.zarr_store import (AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig,  # noqa: E402,F401
                                                    ZarrWriteConfig)
