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
    """Node partition by index blocks (``distributed/graph_partition.py``): a rank evaluates only the edges whose
    receiver lies in its block, exchanges the one-hop sender rows before every layer, and the per-atom results of all
    blocks are concatenated at the end (forces of foreign senders travel back by the reverse exchange first)."""

    kind = StrategyKind.GRAPH_PARTITION

    def __init__(self, config: DomainConfig, group: Any = None) -> None:
        super().__init__(config, group)
        self._dm: Any = None
        self._sharded: Any = None
        self.last_edges_owned = 0

    def run_forward(self, model: Any, batch: Any, spec: MLIPSpec, **kwargs: Any) -> dict:
        """``batch`` is the full (replicated) batch; every rank returns the full outputs (per-atom rows of all blocks
        gathered, system sums reduced)."""
        from nvalchemi_toolkit_b200.distributed.distributed_model import DistributedModel
        from nvalchemi_toolkit_b200.distributed.graph_partition import GraphShardedBatch
        from nvalchemi_toolkit_b200.distributed.halo import all_gather_rows

        cfg = self.config if StrategyKind(self.config.strategy) == StrategyKind.GRAPH_PARTITION else \
            self.config.model_copy(update={"strategy": StrategyKind.GRAPH_PARTITION})
        if self._dm is None or self._dm.model is not model:
            self._dm = DistributedModel(model, cfg, spec, self.group)
        sh = self._sharded
        if sh is None or sh.n_global != batch.num_nodes:
            sh = self._sharded = GraphShardedBatch.from_batch(batch, cfg, self._dm.spec, self.group)
        else:
            lo, hi = sh.partitioner.block(self.rank)
            sh.owned["positions"] = batch.positions[lo:hi]
            if sh.needs_rebuild():
                sh.rebuild()
        self.last_edges_owned = sh.halo.edges_owned
        out = self._dm(sh, **kwargs)
        res: dict[str, Any] = {}
        for key, value in out.items():
            if isinstance(value, torch.Tensor) and value.dim() >= 1 and value.shape[0] == sh.n_owned and sh.n_owned != 1:
                res[key], _ = all_gather_rows(value.contiguous(), self.group)
            else:
                res[key] = value
        return res


_REGISTRY = {StrategyKind.HALO: HaloStrategy, StrategyKind.GRAPH_PARTITION: GraphPartitionStrategy}


def get_strategy(config: DomainConfig, group: Any = None) -> ParallelizationStrategy:
    return _REGISTRY[StrategyKind(config.strategy)](config, group)


def register_strategy(kind: StrategyKind, cls: type) -> None:
    _REGISTRY[kind] = cls
