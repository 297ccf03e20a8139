# SPDX-License-Identifier: Apache-2.0
"""Two-dimensional decomposition: a pipeline of dynamics stages, each stage domain-decomposed over its own ranks.

Reference: the grouped mode of ``DistributedPipeline`` with ``DeviceMesh(("pipeline", "domain"))``
(``nvalchemi/dynamics/base.py:3631-3774,4097-4116``, ``distributed/domain_parallel.py:685-839``): whole systems travel
from stage to stage, inside a stage one large system is split over the ranks of the stage's domain group; only the
lead rank of a group talks to the neighbouring stages; an empty batch travels down the chain as the end marker.

Rank layout: ``rank = stage * domain_size + domain_rank``; the lead of a stage is its ``domain_rank == 0``.
"""
from __future__ import annotations

from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.distributed.config import DomainConfig
from nvalchemi_toolkit_b200.distributed.domain_parallel import DomainParallel


class DomainPipeline:
    """``stage_factories[k]()`` builds the dynamics object of stage ``k`` (called on the ranks of that stage only);
    ``n_steps[k]`` steps are run on every system that passes through the stage."""

    def __init__(self, stage_factories: Sequence[Callable[[], Any]], n_steps: Sequence[int], config: DomainConfig,
                 domain_size: int, template: Batch) -> None:
        if not dist.is_initialized():
            raise RuntimeError("DomainPipeline needs an initialised process group (start with torchrun)")
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.n_stages, self.domain_size = len(stage_factories), int(domain_size)
        if self.world != self.n_stages * self.domain_size:
            raise ValueError(f"world size {self.world} != stages {self.n_stages} x domain size {self.domain_size}")
        self.stage, self.domain_rank = divmod(self.rank, self.domain_size)
        # every rank takes part in the creation of every group
        self.groups = [dist.new_group(list(range(s * self.domain_size, (s + 1) * self.domain_size)))
                       for s in range(self.n_stages)]
        self.group = self.groups[self.stage]
        self.lead = self.stage * self.domain_size
        self.is_lead = self.domain_rank == 0
        self.prev_lead = self.lead - self.domain_size if self.stage > 0 else None
        self.next_lead = self.lead + self.domain_size if self.stage + 1 < self.n_stages else None
        self.dynamics = stage_factories[self.stage]()
        self.steps = int(n_steps[self.stage])
        self.config, self.template = config, template
        self.results: list[Batch] = []
        self.num_processed = 0

    def _conform(self, batch: Batch) -> Batch:
        """The same system with exactly the template's fields (point-to-point transfers post one message per field of
        the template, so sender and receiver must agree on the field set)."""
        from nvalchemi_toolkit_b200.distributed.sharded_batch import _make_batch, _node_fields, _system_fields

        have_n, have_s = _node_fields(batch), _system_fields(batch)
        n = batch.num_nodes
        node = {k: (have_n[k] if k in have_n else v.new_zeros((n,) + tuple(v.shape[1:])))
                for k, v in _node_fields(self.template).items()}
        system = {k: (have_s[k] if k in have_s else v.new_zeros((1,) + tuple(v.shape[1:])))
                  for k, v in _system_fields(self.template).items()}
        return _make_batch(node, system, self.template)

    # ---- inside a stage --------------------------------------------------------------------------------------
    def _replicate(self, batch: Batch | None) -> Batch:
        """Lead → every rank of the stage's domain group (an empty batch is the end marker)."""
        if self.is_lead:
            for r in range(1, self.domain_size):
                batch.send(self.lead + r, tag=100)
            return batch
        return Batch.recv(self.lead, self.template, device=self.template.device, tag=100)

    def _run_stage(self, batch: Batch) -> Batch | None:
        dp = DomainParallel(self.dynamics, self.config, group=self.group)
        self.dynamics.step_count = 0
        if hasattr(self.dynamics, "_state"):
            self.dynamics._state = None  # per-system integrator state starts fresh for every system
        dp.run(batch, n_steps=self.steps)
        out = dp.gather(dst=0)  # group-local rank 0 = lead
        return self._conform(out) if out is not None else None

    # ---- the pipeline ----------------------------------------------------------------------------------------
    def run(self, inputs: Sequence[Batch] | None = None) -> list[Batch]:
        """``inputs`` (single-system batches) are read on the lead of stage 0; finished systems are returned on the
        lead of the last stage (other ranks return an empty list)."""
        empty = self.template.index_select([])
        queue = list(inputs) if (self.stage == 0 and self.is_lead and inputs is not None) else []
        pending = None
        while True:
            if self.is_lead:
                if self.stage == 0:
                    batch = queue.pop(0) if queue else empty
                else:
                    batch = Batch.recv(self.prev_lead, self.template, device=self.template.device, tag=200)
            else:
                batch = None
            batch = self._replicate(batch)
            done = batch.num_graphs == 0
            out = None if done else self._run_stage(batch)
            if self.is_lead:
                if pending is not None:
                    pending.wait()
                    pending = None
                if self.next_lead is not None:
                    pending = (empty if done else out).isend(self.next_lead, tag=200)  # overlaps the next system
                elif not done:
                    self.results.append(out)
            if done:
                break
            self.num_processed += 1
        if pending is not None:
            pending.wait()
        return self.results
