# SPDX-License-Identifier: Apache-2.0
"""Parallelisation strategies behind ``DistributedModel``.

Reference: ``nvalchemi/distributed/strategy.py:71-960`` (``ParallelizationStrategy`` ABC, ``HaloStrategy``,
``GraphPartitionStrategy``, a registry).  ``HaloStrategy`` splits space and exchanges ghost atoms;
``GraphPartitionStrategy`` keeps the geometry replicated on every rank, gives each rank a contiguous block of atoms
whose energies it is responsible for, and all-reduces forces and system sums.  The second one needs no spatial
locality (gas-phase clusters, very small cells) at the price of replicated memory.
"""
from __future__ import annotations

import abc
from types import SimpleNamespace
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.distributed.config import DomainConfig, StrategyKind
from nvalchemi_toolkit_b200.distributed.context import DistributedContext, activate_dd_context
from nvalchemi_toolkit_b200.distributed.halo import _world
from nvalchemi_toolkit_b200.distributed.partitioner import IndexPartitioner
from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec


class ParallelizationStrategy(abc.ABC):
    kind: StrategyKind

    def __init__(self, config: DomainConfig, group: Any = None) -> None:
        self.config, self.group = config, group
        self.rank, self.world = _world(group)

    @abc.abstractmethod
    def run_forward(self, model: Any, batch: Any, spec: MLIPSpec, **kwargs: Any) -> dict: ...

    def reduce_system(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            t = t.clone()
            dist.all_reduce(t, group=self.group)
        return t

    def global_atom_count(self, n_local: int, device: Any = "cpu") -> int:
        return int(self.reduce_system(torch.tensor([n_local], device=device)))


class HaloStrategy(ParallelizationStrategy):
    kind = StrategyKind.HALO

    def __init__(self, config: DomainConfig, group: Any = None) -> None:
        super().__init__(config, group)
        self._dm: Any = None

    def run_forward(self, model: Any, batch: Any, spec: MLIPSpec, **kwargs: Any) -> dict:
        """``batch`` is a ``ShardedBatch``."""
        from nvalchemi_toolkit_b200.distributed.distributed_model import DistributedModel

        if self._dm is None or self._dm.model is not model:
            self._dm = DistributedModel(model, self.config, spec, self.group)
        return self._dm(batch, **kwargs)


class GraphPartitionStrategy(ParallelizationStrategy):
    kind = StrategyKind.GRAPH_PARTITION

    def __init__(self, config: DomainConfig, group: Any = None) -> None:
        super().__init__(config, group)
        self._hook: Any = None

    def run_forward(self, model: Any, batch: Any, spec: MLIPSpec, **kwargs: Any) -> dict:
        """``batch`` is the full (replicated) batch; every rank returns the full, summed outputs."""
        from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook

        n = batch.num_nodes
        lo, hi = IndexPartitioner(n, self.world).block(self.rank)
        nc = model.model_config.neighbor_config
        if nc is not None:
            if self._hook is None:
                self._hook = NeighborListHook(nc, skin=self.config.skin)
            self._hook(SimpleNamespace(batch=batch), None)
        weights = torch.zeros(n, dtype=batch.positions.dtype, device=batch.device)
        weights[lo:hi] = 1.0
        if spec.consolidation == Consolidation.DIRECT_MASKED and nc is not None:
            saved = batch.num_neighbors.clone()
            batch.num_neighbors[:lo] = 0
            batch.num_neighbors[hi:] = 0
        else:
            saved = None
            try:
                batch["energy_weights"] = weights
            except KeyError:
                batch.add_key("energy_weights", weights, level="node", overwrite=True)
        ctx = DistributedContext(self.rank, self.world, hi - lo, n, is_halo=False, is_sharded=True, group=self.group)
        try:
            with activate_dd_context(ctx):
                out = dict(model(batch, **kwargs))
        finally:
            if saved is not None:
                batch.num_neighbors.copy_(saved)
        res: dict[str, Any] = {}
        for key, value in out.items():
            if not isinstance(value, torch.Tensor):
                res[key] = value
                continue
            v = value.detach().clone()
            if key in spec.extensive_outputs or key == "forces":
                if key == "forces" and spec.consolidation == Consolidation.DIRECT_MASKED:
                    v[:lo] = 0
                    v[hi:] = 0
                v = self.reduce_system(v)
            elif v.dim() >= 1 and v.shape[0] == n:  # other per-atom outputs: each rank contributes its block
                block = torch.zeros_like(v)
                block[lo:hi] = v[lo:hi]
                v = self.reduce_system(block)
            res[key] = v
        return res


_REGISTRY = {StrategyKind.HALO: HaloStrategy, StrategyKind.GRAPH_PARTITION: GraphPartitionStrategy}


def get_strategy(config: DomainConfig, group: Any = None) -> ParallelizationStrategy:
    return _REGISTRY[StrategyKind(config.strategy)](config, group)


def register_strategy(kind: StrategyKind, cls: type) -> None:
    _REGISTRY[kind] = cls
