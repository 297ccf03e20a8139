# SPDX-License-Identifier: Apache-2.0
"""``DomainParallel``: run any dynamics object on one system split over ranks.

Reference: ``nvalchemi/distributed/domain_parallel.py:200-975`` and ``_dynamics_coordinator.py:40-170``.  The wrapped
dynamics object keeps integrating an ordinary :class:`Batch` (its rank's owned atoms); this class replaces the model
evaluation with a :class:`DistributedModel` forward, re-partitions when the neighbour skin is exhausted (atoms that left
the sub-domain migrate with all their per-atom fields), installs the cross-rank sums that thermostats and optimisers
need, and runs hooks registered with a :class:`HookScope` on the gathered global batch.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.distributed.config import DomainConfig, HookScope
from nvalchemi_toolkit_b200.distributed.distributed_model import DistributedModel, DistributedPipelineModel
from nvalchemi_toolkit_b200.distributed.halo import _world
from nvalchemi_toolkit_b200.distributed.sharded_batch import ShardedBatch
from nvalchemi_toolkit_b200.distributed.spec import MLIPSpec
from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage
from nvalchemi_toolkit_b200.hooks.core import DynamicsContext


class DynamicsCoordinator:
    """Installs cross-rank reductions into the seams integrators expose (kinetic-energy sum and atom count for
    Nose-Hoover chains, ``v.f / v.v / f.f`` sums and the step-length maximum for FIRE variants)."""

    def __init__(self, dynamics: Any, group: Any = None) -> None:
        self.dynamics, self.group = dynamics, group
        _, self.world = _world(group)
        if self.world == 1:
            return
        for name in ("ke_reduce", "count_reduce", "reduce"):
            if hasattr(dynamics, name):
                setattr(dynamics, name, self.sum)
        if hasattr(dynamics, "reduce_max"):
            dynamics.reduce_max = self.max
        if hasattr(dynamics, "compute_reductions"):
            dynamics.compute_reductions = False

    def sum(self, t: torch.Tensor) -> torch.Tensor:
        t = t.clone()
        dist.all_reduce(t, group=self.group)
        return t

    def max(self, t: torch.Tensor) -> torch.Tensor:
        t = t.clone()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def before_pre_update(self, batch: Batch) -> None:
        """FIRE (first variant) takes its three sums as inputs when it does not compute them itself."""
        dyn = self.dynamics
        if self.world == 1 or not hasattr(dyn, "compute_reductions") or getattr(dyn, "_state", None) is None:
            return
        s = dyn._state
        v, f = batch.velocities.double(), batch.forces.double()
        sums = torch.stack([(v * f).sum(), (v * v).sum(), (f * f).sum()])
        dist.all_reduce(sums, group=self.group)
        for key, val in zip(("vf", "vv", "ff"), sums):
            s[key].copy_(val.to(s[key].dtype).expand_as(s[key]))  # stays on the device: no host read


class DomainParallel:
    """Runs ``dynamics`` on one system split over the ranks of ``group``.

    Usable as a context manager (``with DomainParallel(...) as dp:``); leaving the block releases the peer-mapped
    buffers collectively.  ``async_migration`` (default) decides ghost-list rebuilds and atom migration from a flag that
    was reduced during the previous step, so that no step waits for its own reduction
    (reference ``nvalchemi/distributed/domain_parallel.py:259,313-315,500-524``)."""

    def __init__(self, dynamics: Any, config: DomainConfig, spec: MLIPSpec | None = None, group: Any = None,
                 max_neighbors: int | None = None, async_migration: bool = True) -> None:
        if group is None and config.mesh is not None:
            group = config.mesh.get_group(config.mesh_dim)  # the ranks of the mesh's domain dimension share the system
        self.dynamics, self.config, self.group = dynamics, config, group
        self.rank, self.world = _world(group)
        self.async_migration = bool(async_migration)
        from nvalchemi_toolkit_b200.models.pipeline import PipelineModelWrapper

        if isinstance(dynamics.model, PipelineModelWrapper):
            self.model = DistributedPipelineModel(dynamics.model, config, group, max_neighbors=max_neighbors)
            self.config = config = config.model_copy(update={"ghost_width": max(config.ghost_width,
                                                                                 self.model.required_ghost_width)})
            self.spec = None  # the sharded batch takes its halo width from the config
        else:
            self.model = DistributedModel(dynamics.model, config, spec, group, max_neighbors=max_neighbors)
            self.spec = self.model.spec
        self.coordinator = DynamicsCoordinator(dynamics, group)
        self.sharded: ShardedBatch | None = None
        self._scoped: list[tuple[Any, DynamicsStage, HookScope]] = []
        self.num_rebuilds = 0
        self.converged = False
        self.health_check_every = 64  # steps between reads of the device-side rendezvous status word

    def __enter__(self) -> "DomainParallel":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()

    def close(self) -> None:
        engine = getattr(self.model, "engine", None)
        if engine is not None and engine.p2p is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            engine.p2p = None
            engine._bound = None

    # ---- set-up ---------------------------------------------------------------
    def partition(self, batch: Batch) -> ShardedBatch:
        from nvalchemi_toolkit_b200.distributed.config import StrategyKind

        if StrategyKind(self.config.strategy) == StrategyKind.GRAPH_PARTITION:
            from nvalchemi_toolkit_b200.distributed.graph_partition import GraphShardedBatch

            self.sharded = GraphShardedBatch.from_batch(batch, self.config, self.spec, self.group)
        else:
            self.sharded = ShardedBatch.from_batch(batch, self.config, self.spec, self.group,
                                                   local_periodic=getattr(self.model, "wants_local_periodic", False))
        self._sync_atom_ids()
        return self.sharded

    def _sync_atom_ids(self) -> None:
        """Stochastic integrators draw noise per *global* atom id, so trajectories do not depend on the decomposition."""
        if hasattr(self.dynamics, "atom_ids"):
            self.dynamics.atom_ids = self.sharded.global_ids

    def register_hook(self, hook: Any, stage: DynamicsStage | None = None, scope: HookScope = HookScope.LOCAL) -> None:
        stage = stage if stage is not None else getattr(hook, "stage", DynamicsStage.AFTER_STEP)
        if scope == HookScope.LOCAL:
            self.dynamics.register_hook(hook, stage) if stage is not None else self.dynamics.register_hook(hook)
        else:
            self._scoped.append((hook, stage, scope))

    def _call_scoped(self, stage: DynamicsStage) -> None:
        due = [(h, sc) for h, st, sc in self._scoped
               if st == stage and self.dynamics.step_count % max(1, getattr(h, "frequency", 1)) == 0]
        if not due:
            return
        want_all = any(sc == HookScope.GLOBAL for _, sc in due)
        full = self.sharded.gather(dst=None if want_all else 0)
        for hook, scope in due:
            if scope == HookScope.GLOBAL or self.rank == 0:
                ctx = DynamicsContext(batch=full, step_count=self.dynamics.step_count, model=self.dynamics.model,
                                      converged_mask=None, global_rank=self.rank, workflow=self.dynamics)
                hook(ctx, stage)

    # ---- stepping -------------------------------------------------------------
    def _rebuild(self) -> None:
        self.sharded.rebuild()
        self.num_rebuilds += 1
        self._sync_atom_ids()
        state = getattr(self.dynamics, "_state", None)
        if state is not None and hasattr(self.dynamics, "_on_atoms_migrated"):
            self.dynamics._on_atoms_migrated(self.sharded.owned)

    def compute(self, check_rebuild: bool = True) -> dict:
        """Distributed forward; results are written into the owned batch like ``BaseDynamics.compute`` does."""
        sh, dyn = self.sharded, self.dynamics
        if check_rebuild and sh.needs_rebuild():
            self._rebuild()
        out = self.model(sh)
        dyn._validate_model_outputs(out)
        owned = sh.owned
        for key, attr in dyn._OUTPUT_KEY_TO_BATCH_ATTR.items():
            value = out.get(key)
            if value is None:
                continue
            if attr == "energy" and value.dim() == 1:
                value = value.unsqueeze(-1)
            target = getattr(owned, attr, None)
            if target is not None and target.shape == value.shape and target.dtype == value.dtype:
                target.copy_(value)
            else:
                owned[attr] = value
        dyn._last_outputs = out
        return out

    def _global_convergence(self, owned: Batch) -> bool:
        """Every criterion must hold on every rank's atoms (one small MIN reduction and one host read per check)."""
        hook = self.dynamics.convergence_hook
        if hook is None or self.dynamics.step_count % max(1, hook.frequency) != 0:
            return False
        ok = hook.converged_mask(owned).all().to(torch.int32).reshape(1)
        if self.world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        return bool(int(ok))

    def _fusable_finalize(self) -> bool:
        """The closing velocity update can ride on the force-return kernel of the peer-memory engine: plain half kick,
        float32 contiguous state, and no re-partition inside the compute phase (it would replace the velocity tensor)."""
        engine = getattr(self.model, "engine", None)
        if engine is None or not self.config.fuse_integrator_finalize or not self.async_migration:
            return False
        if not getattr(self.dynamics, "__dd_half_kick_finalize__", False) or not getattr(engine, "fused_force_return", False):
            return False
        owned, state = self.sharded.owned, getattr(self.dynamics, "_state", None) or {}
        v, m, dt = getattr(owned, "velocities", None), getattr(owned, "atomic_masses", None), state.get("dt")
        return (v is not None and m is not None and dt is not None and v.dtype == torch.float32 and v.is_contiguous()
                and m.dtype == torch.float32 and dt.dtype == torch.float32 and owned.batch_idx.dtype == torch.int32)

    def step(self) -> ShardedBatch:
        sh, dyn = self.sharded, self.dynamics
        fuse = False
        if sh is None:
            raise RuntimeError("call partition(batch) first")
        if self.async_migration and sh.consume_rebuild_check():
            self._rebuild()  # may replace sh.owned (migration)
        dyn._ensure_state_initialized(sh.owned)
        for stage, fn in ((DynamicsStage.BEFORE_STEP, None), (DynamicsStage.BEFORE_PRE_UPDATE, "pre"),
                          (DynamicsStage.AFTER_PRE_UPDATE, None), (DynamicsStage.BEFORE_COMPUTE, "compute"),
                          (DynamicsStage.AFTER_COMPUTE, None), (DynamicsStage.BEFORE_POST_UPDATE, "post"),
                          (DynamicsStage.AFTER_POST_UPDATE, None), (DynamicsStage.AFTER_STEP, None)):
            dyn._call_hooks(stage, sh.owned)
            self._call_scoped(stage)
            if fn == "pre":
                self.coordinator.before_pre_update(sh.owned)
                dyn.pre_update(sh.owned)
                if self.async_migration:
                    sh.dispatch_rebuild_check()  # positions are final for this step; the flag is read at the next one
            elif fn == "compute":
                fuse = self._fusable_finalize()
                if fuse:
                    owned = sh.owned
                    self.model.engine.fused_finalize = (owned.velocities, owned.atomic_masses, dyn._state["dt"], owned.batch_idx)
                try:
                    self.compute(check_rebuild=not self.async_migration)
                finally:
                    if fuse:
                        self.model.engine.fused_finalize = None
            elif fn == "post":
                if not fuse:  # else the force-return kernel already applied the closing half kick
                    dyn.post_update(sh.owned)
        self.converged = self._global_convergence(sh.owned)
        if self.converged:
            dyn._call_hooks(DynamicsStage.ON_CONVERGE, sh.owned)
            self._call_scoped(DynamicsStage.ON_CONVERGE)
        dyn.step_count += 1
        engine = getattr(self.model, "engine", None)
        if engine is not None and dyn.step_count % self.health_check_every == 0:
            engine.check()
        return sh

    def run(self, batch: Batch | ShardedBatch | None = None, n_steps: int | None = None) -> ShardedBatch:
        if isinstance(batch, ShardedBatch):
            self.sharded = batch
            self._sync_atom_ids()
        elif batch is not None:
            self.partition(batch)
        n = n_steps if n_steps is not None else self.dynamics.n_steps
        if n is None:
            raise ValueError("No step count provided")
        if getattr(self.sharded.owned, "forces", None) is None or self.dynamics.step_count == 0:
            self.compute()  # integrators need forces at the first half-kick
        self.dynamics._open_hooks()
        try:
            for _ in range(n):
                self.step()
                if self.converged:
                    break
        finally:
            self.dynamics._close_hooks()
        return self.sharded

    def gather(self, dst: int | None = None) -> Batch | None:
        return self.sharded.gather(dst)
