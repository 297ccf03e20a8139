# SPDX-License-Identifier: Apache-2.0
"""``DistributedPipeline``: one dynamics stage per rank, graduated systems handed to the next rank.

Behaviour follows the reference (``nvalchemi/dynamics/base.py:3340-4189``): ``a | b`` builds a two-stage pipeline,
further ``|`` appends; the first stage feeds itself from a :class:`SizeAwareSampler` (inflight batching); every
iteration each stage posts a receive from its predecessor, steps its active batch, and sends its graduated systems
(an empty batch when there are none, so a posted receive always completes); the final stage writes graduated systems to
its sinks; termination is agreed with an ``all_reduce(MAX)`` over per-stage done flags.  The hand-off stays on
``torch.distributed`` point-to-point messages (NCCL on GPUs, Gloo on CPU) and is overlapped with the stage's compute:
the receive is posted before the step and completed after it, the send is waited for at the start of the next
iteration.  Received systems are merged into the active batch with tensor concatenation (no per-system Python
objects).
"""
from __future__ import annotations

import os
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.dynamics.base import BaseDynamics, BufferConfig, DynamicsStage, _flat_status
from nvalchemi_toolkit_b200.dynamics.sinks import strip_neighbor_caches


class DistributedPipeline:
    def __init__(self, stages: dict[int, BaseDynamics], synchronized: bool = False, debug_mode: bool = False,
                 mesh: Any = None, group: Any = None, **dist_kwargs: Any) -> None:
        """``stages`` maps a (global) rank to its dynamics stage.  ``group``: process group that holds exactly the ranks
        of this pipeline, for jobs that run several independent pipelines side by side (lanes); template broadcast and
        the termination vote then stay inside the lane."""
        self.stages = dict(sorted(stages.items()))
        self.group = group
        self.synchronized = synchronized
        self.debug_mode = debug_mode
        self.mesh = mesh
        self.dist_kwargs = dist_kwargs
        self._owns_pg = False
        self._template: Batch | None = None
        self._pending_send: Any = None
        self.iterations = 0
        self._done_flags: torch.Tensor | None = None
        self._is_setup = False

    # ---- composition -----------------------------------------------------------
    def __or__(self, other: "BaseDynamics | DistributedPipeline") -> "DistributedPipeline":
        stages = dict(self.stages)
        nxt = max(stages) + 1
        if isinstance(other, DistributedPipeline):
            for k, st in other.stages.items():
                stages[nxt + k] = st
        else:
            stages[nxt] = other
        return DistributedPipeline(stages, self.synchronized, self.debug_mode, self.mesh, self.group, **self.dist_kwargs)

    # ---- lifecycle ---------------------------------------------------------------
    def init_distributed(self) -> None:
        if dist.is_initialized():
            return
        backend = self.dist_kwargs.get("backend") or ("nccl" if torch.cuda.is_available() else "gloo")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kwargs = {k: v for k, v in self.dist_kwargs.items() if k != "backend"}
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend, **kwargs)
        self._owns_pg = True

    def __enter__(self) -> "DistributedPipeline":
        self.init_distributed()
        self.setup()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._owns_pg and dist.is_initialized():
            dist.destroy_process_group()
            self._owns_pg = False

    @property
    def rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    @property
    def stage(self) -> BaseDynamics | None:
        return self.stages.get(self.rank)

    def setup(self) -> None:
        """Wire neighbour ranks, allocate hand-off templates, share the batch template with every stage."""
        ranks = list(self.stages)
        world = dist.get_world_size() if dist.is_initialized() else 1
        if max(ranks) >= world:
            raise ValueError(f"pipeline has a stage for rank {max(ranks)} but the world size is {world}")
        for i, r in enumerate(ranks):
            st = self.stages[r]
            st.prior_rank = ranks[i - 1] if i > 0 else None
            st.next_rank = ranks[i + 1] if i + 1 < len(ranks) else None
            if st.buffer_config is None:
                st.buffer_config = BufferConfig(num_systems=st.max_batch_size, num_nodes=0, num_edges=0)
        self._done_flags = None
        self._share_templates()
        self._is_setup = True

    def _share_templates(self) -> None:
        """The first stage knows the batch layout (from its sampler or active batch); everyone receives an empty copy."""
        ranks = list(self.stages)
        first = ranks[0]
        payload: list[Any] = [None]
        if self.rank == first:
            st = self.stages[first]
            if st.active_batch is None and st.sampler is not None:
                st.active_batch = st.sampler.build_initial_batch()
                dev = self._device(st)
                if st.active_batch.device != dev:  # datasets live on the host; the stage runs on its device
                    st.active_batch = st.active_batch.to(dev)
            if st.active_batch is None:
                raise RuntimeError("first pipeline stage needs a sampler or an active batch")
            st._ensure_bookkeeping_fields(st.active_batch)
            for _, d in getattr(st, "sub_stages", []):
                pass
            payload = [st.active_batch.index_select(torch.zeros(0, dtype=torch.long)).to("cpu")]
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast_object_list(payload, src=first, group=self.group)
        self._template = payload[0]

    # ---- one iteration -------------------------------------------------------------
    def _device(self, st: BaseDynamics) -> torch.device:
        if dist.is_initialized() and dist.get_backend() == "gloo":
            return torch.device("cpu")
        return st.device

    def _graduated_mask(self, st: BaseDynamics, batch: Batch, converged: torch.Tensor | None) -> torch.Tensor:
        m = torch.zeros(batch.num_graphs, dtype=torch.bool, device=batch.device)
        if converged is not None:
            m[converged] = True
        status = _flat_status(batch)
        if status is not None and hasattr(st, "sub_stages"):
            m |= status >= st.exit_status
        if st.convergence_hook is None and st.n_steps is not None and not hasattr(st, "sub_stages"):
            key = "pipeline_steps"
            if getattr(batch, key, None) is None:
                batch.add_key(key, torch.zeros(batch.num_graphs, 1, dtype=torch.long, device=batch.device), "system")
            cnt = getattr(batch, key).reshape(-1)
            cnt += 1
            m |= cnt >= st.n_steps
        return m

    def step(self) -> None:
        st = self.stage
        if st is None:
            return
        dev = self._device(st)
        template = self._template.to(dev)
        if self._pending_send is not None:
            self._pending_send.wait()
            self._pending_send = None
        # comm_mode of the stage: "sync" completes the receive before the step and the send right after posting it (no
        # overlap, simplest to reason about); "async_recv" overlaps the receive with the step but completes the send at
        # once; "fully_async" also leaves the send in flight until the start of the next iteration
        mode = getattr(st, "comm_mode", "fully_async")
        recv = Batch.irecv(st.prior_rank, template, device=dev) if st.prior_rank is not None else None
        early: Batch | None = None
        if recv is not None and mode == "sync":
            early, recv = recv.wait(), None
        graduated: Batch | None = None
        batch = st.active_batch
        if batch is not None and batch.num_graphs > 0:
            if getattr(st, "_primed_for", None) is not batch:
                st._ensure_bookkeeping_fields(batch)
                st._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
                for _, d in getattr(st, "sub_stages", []):
                    d._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
                st.compute(batch)
                st._primed_for = batch
            batch, converged = st.step(batch)
            mask = self._graduated_mask(st, batch, converged)
            if bool(mask.any()):
                graduated = strip_neighbor_caches(batch.index_select(mask))  # messages carry the template's fields only
                rest = batch.index_select(~mask) if not bool(mask.all()) else None
                st._sync_state_to_batch(torch.nonzero(~mask).squeeze(1), 0, rest if rest is not None else batch)
                batch = rest
            st.active_batch = batch
            st._primed_for = batch if graduated is None else None
        if recv is not None or early is not None:
            incoming = early if early is not None else recv.wait()
            if incoming.num_graphs:
                n_old = st.active_batch.num_graphs if st.active_batch is not None else 0
                st._recv_to_batch(self._strip(incoming, st))
                n_new = (st.active_batch.num_graphs if st.active_batch is not None else 0) - n_old
                if n_new > 0:
                    st._sync_state_to_batch(torch.arange(n_old, device=dev), n_new, st.active_batch)
                    st._primed_for = None
        if st.next_rank is not None:
            out = graduated if graduated is not None else template
            self._pending_send = out.isend(st.next_rank, template=template)
            self._keepalive = out
            if mode != "fully_async":
                self._pending_send.wait()
                self._pending_send = None
        elif graduated is not None and st.sinks:
            st._overflow_to_sinks(graduated)
        elif graduated is not None:
            self.finished = getattr(self, "finished", [])
            self.finished.append(graduated.to("cpu"))
        if st.prior_rank is None and st.sampler is not None:
            self._refill(st, dev)
        self.iterations += 1

    @staticmethod
    def _strip(incoming: Batch, st: BaseDynamics) -> Batch:
        """Reset per-stage bookkeeping of systems arriving from the previous stage."""
        if getattr(incoming, "status", None) is not None:
            incoming.status.zero_()
        for key in list(incoming._storage.keys()):
            if key.startswith("n_steps_counter_") or key == "pipeline_steps":
                incoming[key].zero_()
        return incoming

    def _refill(self, st: BaseDynamics, dev: torch.device) -> None:
        s = st.sampler
        batch = st.active_batch
        n = batch.num_graphs if batch is not None else 0
        atoms = batch.num_nodes if batch is not None else 0
        edges = batch.num_edges if batch is not None else 0
        repl = s.request_replacements_budget(
            atom_budget=None if s.max_atoms is None else s.max_atoms - atoms,
            edge_budget=None if s.max_edges is None else s.max_edges - edges,
            max_count=(s.max_batch_size if s.max_batch_size is not None else st.max_batch_size) - n)
        if not repl:
            return
        new = Batch.from_data_list(repl, device=dev)
        st._ensure_bookkeeping_fields(new)
        if batch is None:
            st.active_batch = new
            st._state = None
        else:
            for key in list(batch._storage.keys()):
                if key not in new:
                    ref, lvl = batch[key], batch._storage.group_of(key)
                    rows = {"atoms": new.num_nodes, "edges": new.num_edges, "system": new.num_graphs}[lvl]
                    new.add_key(key, ref.new_zeros((rows,) + tuple(ref.shape[1:])),
                                level={"atoms": "node", "edges": "edge", "system": "system"}[lvl])
            batch.append(new)
            st._sync_state_to_batch(torch.arange(n, device=dev), new.num_graphs, batch)
        st._primed_for = None

    def _stage_done(self, st: BaseDynamics, prior_done: bool) -> bool:
        empty = st.active_batch is None or st.active_batch.num_graphs == 0
        if st.prior_rank is None:
            source_done = st.sampler is None or st.sampler.exhausted
        else:
            source_done = prior_done
        return bool(empty and source_done)

    def _sync_done_flags(self) -> bool:
        ranks = list(self.stages)
        dev = self._device(self.stage) if self.stage is not None else torch.device("cpu")
        if self._done_flags is None:
            self._done_flags = torch.zeros(len(ranks), dtype=torch.int32, device=dev)
        st = self.stage
        if st is not None:
            i = ranks.index(self.rank)
            prior_done = i == 0 or bool(self._done_flags[i - 1])
            # a stage may only finish one iteration after its predecessor: its last send is then already received
            self._done_flags[i] = int(self._stage_done(st, prior_done))
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(self._done_flags, op=dist.ReduceOp.MAX, group=self.group)
        return bool(self._done_flags.all())

    def run(self, max_iterations: int | None = None) -> None:
        if not self._is_setup:
            self.setup()
        st = self.stage
        if st is not None:
            st._open_hooks()
        try:
            while True:
                self.step()
                if self._sync_done_flags():
                    break
                if max_iterations is not None and self.iterations >= max_iterations:
                    break
        finally:
            if self._pending_send is not None:
                self._pending_send.wait()
                self._pending_send = None
            if st is not None:
                st._close_hooks()
            if self.synchronized and dist.is_initialized():
                dist.barrier(group=self.group)
