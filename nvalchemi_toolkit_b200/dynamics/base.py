# SPDX-License-Identifier: Apache-2.0
"""Dynamics engine: the nine-stage step loop, convergence, stage fusion (``+``) and pipelining (``|``).

Behaviour follows the reference's ``nvalchemi/dynamics/base.py``:

* ``DynamicsStage`` values and ordering (``:120-157``);
* ``BaseDynamics.step`` = hooks → ``pre_update`` → hooks → ``compute`` → hooks → ``post_update`` →
  hooks → convergence (``:1815-1902``); systems whose ``status >= exit_status`` are frozen;
* ``compute`` writes model outputs into the batch, detaches them and clears ``requires_grad``
  (``:1718-1813``);
* ``ConvergenceHook`` with AND-ed criteria and optional status migration (``:160-349, 2215-2501``);
* ``FusedStage``: one model evaluation shared by several integrators selected per system through the
  ``status`` key, ``n_steps`` budgets per sub-stage, inflight refill through a sampler
  (``:2504-3337``);
* ``a + b`` → ``FusedStage``; ``a | b`` → ``DistributedPipeline`` (``:1184-1243``).

The pipeline itself lives in :mod:`nvalchemi_toolkit_b200.dynamics.pipeline`.
"""
from __future__ import annotations

from collections import OrderedDict
from enum import Enum
from typing import Any, Callable, ClassVar, Literal, Sequence

import torch
import torch.distributed as dist
from pydantic import BaseModel, ConfigDict, Field

from nvalchemi_toolkit_b200.data.batch import Batch
from nvalchemi_toolkit_b200.hooks.core import DynamicsContext, HookRegistryMixin
from nvalchemi_toolkit_b200.models.base import BaseModelMixin


class BufferConfig(BaseModel):
    """Capacity of the pre-allocated send/receive buffers of a pipeline stage."""

    num_systems: int = Field(ge=0)
    num_nodes: int = Field(ge=0)
    num_edges: int = Field(ge=0)


class DynamicsStage(Enum):
    BEFORE_STEP = 0
    BEFORE_PRE_UPDATE = 1
    AFTER_PRE_UPDATE = 2
    BEFORE_COMPUTE = 3
    AFTER_COMPUTE = 4
    BEFORE_POST_UPDATE = 5
    AFTER_POST_UPDATE = 6
    AFTER_STEP = 7
    ON_CONVERGE = 8


def _flat_status(batch: Batch) -> torch.Tensor | None:
    s = getattr(batch, "status", None)
    if s is None:
        return None
    return s.reshape(-1)[: batch.num_graphs] if s.dim() == 2 else s[: batch.num_graphs]


class _ConvergenceCriterion(BaseModel):
    """``reduce(batch[key]) <= threshold`` per system; node-level values are max-reduced per graph."""

    model_config = ConfigDict(arbitrary_types_allowed=True)
    key: str
    threshold: float = 0.0
    reduce_dims: int | list[int] = -1
    reduce_op: Literal["min", "max", "norm", "mean", "sum"] | None = None
    custom_op: Callable[[torch.Tensor], torch.Tensor] | None = None

    def _reduce(self, t: torch.Tensor) -> torch.Tensor:
        op, dims = self.reduce_op, self.reduce_dims
        if op is None:
            return t
        if op == "min":
            return torch.amin(t, dims)
        if op == "max":
            return torch.amax(t, dims)
        if op == "norm":
            return torch.linalg.vector_norm(t, dim=dims)
        if op == "mean":
            return torch.mean(t, dim=dims)
        return torch.sum(t, dim=dims)

    def __call__(self, batch: Batch) -> torch.Tensor:
        target = getattr(batch, self.key, None)
        if target is None:
            raise KeyError(f"Key for convergence check not found; expected={self.key!r}, "
                           f"available={list(batch.model_dump(exclude_none=True))}")
        if self.custom_op is not None:
            return self.custom_op(target)
        target = self._reduce(target)
        if target.shape[0] == batch.num_nodes and batch.num_nodes != batch.num_graphs:
            if target.dim() > 1:
                target = target.reshape(target.shape[0], -1).amax(dim=-1)
            from nvalchemi_toolkit_b200.dynamics._ops import segmented_max

            reduced = segmented_max(target.contiguous(), batch.batch_idx, batch.num_graphs)
        else:
            reduced = target.squeeze(-1) if target.dim() == 2 else target
        return reduced <= self.threshold


class ConvergenceHook:
    """AND of criteria per system; optionally migrates ``status`` from ``source`` to ``target``."""

    def __init__(self, criteria: Any = None, source_status: int | None = None, target_status: int | None = None,
                 frequency: int = 1) -> None:
        self.frequency = frequency
        self.stage = DynamicsStage.AFTER_STEP
        self.source_status, self.target_status = source_status, target_status
        if criteria is None:
            criteria = [{"key": "forces", "threshold": 0.05, "reduce_op": "norm", "reduce_dims": -1}]
        if isinstance(criteria, (dict, _ConvergenceCriterion)):
            criteria = [criteria]
        if not isinstance(criteria, (list, tuple)):
            raise TypeError(f"criteria must be a dict, _ConvergenceCriterion, or list thereof, got {type(criteria).__name__}")
        self.criteria: list[_ConvergenceCriterion] = []
        for c in criteria:
            if isinstance(c, dict):
                c = _ConvergenceCriterion(**c)
            if not isinstance(c, _ConvergenceCriterion):
                raise TypeError(f"Each criterion must be a dict or _ConvergenceCriterion, got {type(c).__name__}")
            self.criteria.append(c)

    @classmethod
    def from_forces(cls, threshold: float, frequency: int = 1, source_status: int | None = None,
                    target_status: int | None = None) -> "ConvergenceHook":
        return cls([{"key": "forces", "threshold": threshold, "reduce_op": "norm", "reduce_dims": -1}],
                   source_status, target_status, frequency)

    @classmethod
    def from_fmax(cls, threshold: float = 0.05, source_status: int | None = None, target_status: int | None = None,
                  frequency: int = 1) -> "ConvergenceHook":
        return cls.from_forces(threshold, frequency, source_status, target_status)

    @property
    def num_criteria(self) -> int:
        return len(self.criteria)

    def converged_mask(self, batch: Batch) -> torch.Tensor:
        mask = torch.ones(batch.num_graphs, dtype=torch.bool, device=batch.device)
        for c in self.criteria:
            mask &= c(batch)
        return mask

    def evaluate(self, batch: Batch) -> torch.Tensor | None:
        mask = self.converged_mask(batch)
        if not bool(mask.any()):
            return None
        return torch.where(mask)[0]

    def __call__(self, ctx: DynamicsContext, stage: Enum) -> None:
        batch = ctx.batch
        if self.source_status is None or self.target_status is None:
            return
        status = _flat_status(batch)
        if status is None:
            return
        migrate = self.converged_mask(batch) & (status == self.source_status)
        status.masked_fill_(migrate, self.target_status)

    def __repr__(self) -> str:
        return (f"ConvergenceHook(criteria={self.criteria}, source_status={self.source_status}, "
                f"target_status={self.target_status}, frequency={self.frequency})")


class _CommunicationMixin:
    """Inter-stage plumbing: neighbour ranks, sinks, sampler, send/receive buffers."""

    def __init__(self, *, prior_rank: int | None = -1, next_rank: int | None = -1, sinks: Sequence[Any] | None = None,
                 active_batch: Batch | None = None, max_batch_size: int = 100, done: bool = False,
                 sampler: Any = None, refill_frequency: int = 1, device_type: str | None = None,
                 comm_mode: str = "async_recv", buffer_config: BufferConfig | dict | None = None,
                 debug_mode: bool = False, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        self.prior_rank = None if prior_rank in (-1, None) else prior_rank
        self.next_rank = None if next_rank in (-1, None) else next_rank
        self.sinks = list(sinks) if sinks is not None else []
        self.active_batch = active_batch
        self.max_batch_size = max_batch_size
        self.done = done
        self.sampler = sampler
        self.refill_frequency = refill_frequency
        self.device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        if comm_mode not in ("sync", "async_recv", "fully_async"):
            raise ValueError(f"Invalid comm_mode={comm_mode!r}. Expected one of: 'sync', 'async_recv', 'fully_async'.")
        self.comm_mode = comm_mode
        if isinstance(buffer_config, dict):
            buffer_config = BufferConfig(**buffer_config)
        if buffer_config is not None and not isinstance(buffer_config, BufferConfig):
            raise TypeError(f"Buffer configuration invalid; got a {type(buffer_config)} object.")
        self.buffer_config = buffer_config
        if self.has_neighbor and buffer_config is None:
            raise ValueError("buffer_config is required when prior_rank or next_rank is set. Pre-allocated buffers "
                             "are mandatory for inter-rank communication.")
        self.send_buffer: Batch | None = None
        self.recv_buffer: Batch | None = None
        self._recv_template: Batch | None = None
        self._pending_recv_handle: Any = None
        self._pending_send_handle: Any = None
        self.debug_mode = debug_mode
        self.comm_group: Any = None

    @property
    def has_neighbor(self) -> bool:
        return self.prior_rank is not None or self.next_rank is not None

    @property
    def is_first_stage(self) -> bool:
        return self.prior_rank is None

    @property
    def is_final_stage(self) -> bool:
        return self.next_rank is None

    @property
    def global_rank(self) -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    @property
    def device(self) -> torch.device:
        if self.device_type == "cuda":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device(self.device_type)

    @property
    def room_in_active_batch(self) -> int:
        return self.max_batch_size - (self.active_batch.num_graphs if self.active_batch is not None else 0)

    def _overflow_to_sinks(self, batch: Batch, mask: torch.Tensor | None = None) -> None:
        for sink in self.sinks:
            if not sink.is_full:
                sink.write(batch, mask=mask)
                return
        raise RuntimeError(f"All sinks are full. Cannot store {batch.num_graphs} overflow samples.")

    def _recv_to_batch(self, incoming: Batch) -> None:
        """Merge received systems into the active batch (tensor-level append, no per-system Python objects)."""
        if incoming.num_graphs == 0:
            return
        room = self.room_in_active_batch
        if room <= 0:
            self._overflow_to_sinks(incoming)
            return
        n = incoming.num_graphs
        fit = incoming if n <= room else incoming.index_select(slice(0, room))
        if self.active_batch is None:
            self.active_batch = fit._tight().clone()
        else:
            self.active_batch.append(fit)
        if n > room:
            self._overflow_to_sinks(incoming.index_select(slice(room, n)))

    def _drain_sinks_to_batch(self) -> None:
        for sink in self.sinks:
            room = self.room_in_active_batch
            if room <= 0:
                return
            if len(sink) > 0 and getattr(sink, "drainable", True):
                got = sink.drain(max_systems=room) if "max_systems" in sink.drain.__code__.co_varnames else sink.drain()
                if got is not None and got.num_graphs:
                    self._recv_to_batch(got.to(self.device))


class BaseDynamics(HookRegistryMixin, _CommunicationMixin):
    """Base class of integrators and optimisers: subclasses implement ``pre_update`` / ``post_update``."""

    __needs_keys__: ClassVar[set[str]] = {"forces"}
    __provides_keys__: ClassVar[set[str]] = set()
    _stage_type = DynamicsStage
    _OUTPUT_KEY_TO_BATCH_ATTR: ClassVar[dict[str, str]] = {"energy": "energy", "forces": "forces", "stress": "stress",
                                                          "virial": "virial", "charges": "charges"}
    _mutable_fields: ClassVar[tuple[str, ...]] = ("positions", "velocities", "cell")
    _bookkeeping_keys: ClassVar[dict[str, Callable[[int, torch.device], torch.Tensor]]] = {
        "status": lambda n, dev: torch.zeros(n, 1, dtype=torch.long, device=dev),
        "system_id": lambda n, dev: torch.full((n, 1), -1, dtype=torch.long, device=dev),
    }

    def __init__(self, model: BaseModelMixin, hooks: list | None = None, convergence_hook: Any = None,
                 n_steps: int | None = None, exit_status: int = 1, **kwargs: Any) -> None:
        super().__init__(**kwargs)
        if not isinstance(model, BaseModelMixin):
            raise TypeError(f"Expected a `BaseModelMixin` instance, got {type(model).__name__}. Please wrap your "
                            "model with a `BaseModelMixin` subclass.")
        self.model = model
        if isinstance(model, torch.nn.Module):
            model.eval()  # dynamics is inference: wrappers with hand-written kernels only use them outside training mode
        self.step_count = 0
        if isinstance(convergence_hook, dict):
            convergence_hook = ConvergenceHook(**convergence_hook)
        self.convergence_hook = convergence_hook
        self.n_steps = n_steps
        self.exit_status = exit_status
        self.model_config = model.model_config
        self._last_converged: torch.Tensor | None = None
        self._last_outputs: dict | None = None
        self._init_hooks(hooks)

    @classmethod
    def register_bookkeeping_key(cls, key: str, default_fn: Callable[[int, torch.device], torch.Tensor]) -> None:
        BaseDynamics._bookkeeping_keys = {**BaseDynamics._bookkeeping_keys, key: default_fn}

    # ---- subclass interface ------------------------------------------------
    def pre_update(self, batch: Batch) -> None:  # pragma: no cover - interface
        pass

    def post_update(self, batch: Batch) -> None:  # pragma: no cover - interface
        pass

    def _init_state(self, batch: Batch) -> None:
        pass

    def _make_new_state(self, n: int, template_batch: Batch) -> dict[str, torch.Tensor] | None:
        return None

    def _ensure_state_initialized(self, batch: Batch) -> None:
        st = getattr(self, "_state", None)
        if st is None or (isinstance(st, dict) and st and next(iter(st.values())).shape[0] != batch.num_graphs):
            self._init_state(batch)

    def _sync_state_to_batch(self, remaining_indices: torch.Tensor, n_new: int, template_batch: Batch) -> None:
        """Per-system integrator state follows the systems through refills: keep rows of remaining
        systems, append freshly initialised rows for replacements."""
        st = getattr(self, "_state", None)
        if not isinstance(st, dict) or not st:
            return
        new = self._make_new_state(n_new, template_batch) if n_new > 0 else None
        out = {}
        for k, v in st.items():
            parts = [v[remaining_indices]] if remaining_indices.numel() else []
            if new is not None:
                parts.append(new[k])
            out[k] = torch.cat(parts) if parts else v[:0]
        self._state = out

    # ---- hooks ---------------------------------------------------------------
    def _build_context(self, batch: Batch) -> DynamicsContext:
        mask = None
        if self._last_converged is not None and batch is not None:
            mask = torch.zeros(batch.num_graphs, dtype=torch.bool, device=batch.device)
            idx = self._last_converged
            if idx.numel() and int(idx.max()) >= batch.num_graphs:
                idx = idx[:0]  # the batch was refilled or compacted since; the old indices name other systems
                self._last_converged = None
            mask[idx] = True
        return DynamicsContext(batch=batch, step_count=self.step_count, model=self.model, converged_mask=mask,
                               global_rank=self.global_rank, workflow=self)

    def _check_convergence(self, batch: Batch) -> torch.Tensor | None:
        return None if self.convergence_hook is None else self.convergence_hook.evaluate(batch)

    def _validate_model_outputs(self, outputs: dict) -> None:
        for key in self.__needs_keys__:
            if outputs.get(key) is None:
                raise RuntimeError(f"{type(self).__name__} requires '{key}' (declared in __needs_keys__), but the "
                                   f"model did not produce it. Check the model's ModelConfig to ensure '{key}' is "
                                   "supported and enabled, or that no hooks are missing.")

    # ---- compute ---------------------------------------------------------------
    def compute(self, batch: Batch) -> dict:
        """Model forward; outputs are written into the batch in place and detached."""
        self._last_outputs = None
        outputs = self.model(batch)
        self._validate_model_outputs(outputs)
        detached: "OrderedDict[str, Any]" = OrderedDict(
            (k, v.detach() if isinstance(v, torch.Tensor) else v) for k, v in outputs.items())
        del outputs
        for out_key, attr in self._OUTPUT_KEY_TO_BATCH_ATTR.items():
            value = detached.get(out_key)
            if value is None:
                continue
            target = getattr(batch, attr, None)
            if target is not None and target.shape[0] == value.reshape(target.shape[0], -1).shape[0] \
                    and target.numel() == value.numel():
                target.copy_(value.reshape(target.shape))
            else:
                batch[attr] = value if attr != "energy" or value.dim() == 2 else value.unsqueeze(-1)
        cfg = self.model_config
        grad_keys = {"positions"} | set(cfg.gradient_keys)
        if cfg.autograd_outputs & set(cfg.active_outputs):
            grad_keys |= set(cfg.autograd_inputs)
        for key in grad_keys:
            value = getattr(batch, key, None)
            if isinstance(value, torch.Tensor) and value.requires_grad:
                value.requires_grad_(False)
        self._last_outputs = detached
        return detached

    # ---- step / run ----------------------------------------------------------
    def _frozen_snapshot(self, batch: Batch, active: torch.Tensor) -> tuple[dict, torch.Tensor, torch.Tensor]:
        node_mask = torch.repeat_interleave(active, batch.num_nodes_per_graph.long(), output_size=batch.num_nodes)
        saved = {}
        for f in self._mutable_fields:
            val = getattr(batch, f, None)
            if val is None:
                continue
            if val.shape[0] == batch.num_nodes and batch.num_nodes != batch.num_graphs:
                saved[f] = val[~node_mask].clone()
            elif val.shape[0] == batch.num_graphs:
                saved[f] = val[~active].clone()
        return saved, node_mask, ~active

    def _restore_frozen(self, batch: Batch, saved: dict, node_mask: torch.Tensor, sys_mask: torch.Tensor) -> None:
        with torch.no_grad():
            for f, sv in saved.items():
                val = getattr(batch, f)
                if val.shape[0] == batch.num_nodes and batch.num_nodes != batch.num_graphs:
                    val[~node_mask] = sv
                else:
                    val[sys_mask] = sv

    def step(self, batch: Batch) -> tuple[Batch, torch.Tensor | None]:
        self._ensure_state_initialized(batch)
        self._call_hooks(DynamicsStage.BEFORE_STEP, batch)
        status = _flat_status(batch)
        frozen = None
        if status is not None:
            active = status < self.exit_status
            frozen = self._frozen_snapshot(batch, active)
        self._call_hooks(DynamicsStage.BEFORE_PRE_UPDATE, batch)
        self.pre_update(batch)
        self._call_hooks(DynamicsStage.AFTER_PRE_UPDATE, batch)
        self._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
        self.compute(batch)
        self._call_hooks(DynamicsStage.AFTER_COMPUTE, batch)
        self._call_hooks(DynamicsStage.BEFORE_POST_UPDATE, batch)
        self.post_update(batch)
        self._call_hooks(DynamicsStage.AFTER_POST_UPDATE, batch)
        if frozen is not None:
            self._restore_frozen(batch, *frozen)
        self._call_hooks(DynamicsStage.AFTER_STEP, batch)
        converged = self._check_convergence(batch)
        self._last_converged = converged
        if converged is not None:
            self._call_hooks(DynamicsStage.ON_CONVERGE, batch)
        self.step_count += 1
        return batch, converged

    def masked_update(self, batch: Batch, mask: torch.Tensor) -> None:
        self._ensure_state_initialized(batch)
        frozen = self._frozen_snapshot(batch, mask)
        self.pre_update(batch)
        self.post_update(batch)
        self._restore_frozen(batch, *frozen)

    def _masked_pre_update(self, batch: Batch, mask: torch.Tensor) -> None:
        self._ensure_state_initialized(batch)
        frozen = self._frozen_snapshot(batch, mask)
        self.pre_update(batch)
        self._restore_frozen(batch, *frozen)

    def _masked_post_update(self, batch: Batch, mask: torch.Tensor) -> None:
        frozen = self._frozen_snapshot(batch, mask)
        self.post_update(batch)
        self._restore_frozen(batch, *frozen)

    def run(self, batch: Batch, n_steps: int | None = None) -> Batch:
        resolved = n_steps if n_steps is not None else self.n_steps
        if resolved is None:
            raise ValueError("No step count provided. Either pass `n_steps` to run() or set it at construction time "
                             f"via `{type(self).__name__}(..., n_steps=N)`.")
        self._open_hooks()
        try:
            if "forces" in getattr(self, "__needs_keys__", ()) and getattr(batch, "forces", None) is None:
                # a batch that never saw the model (freshly built from raw coordinates): the first half-kick needs forces
                self._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
                self.compute(batch)
            for _ in range(resolved):
                batch, conv = self.step(batch)
                if self.sampler is None and conv is not None and conv.numel() == batch.num_graphs:
                    break
        finally:
            self._close_hooks()
        return batch

    # ---- inflight batching ---------------------------------------------------
    def _ensure_bookkeeping_fields(self, batch: Batch) -> None:
        for key, fn in self._bookkeeping_keys.items():
            if getattr(batch, key, None) is None:
                batch.add_key(key, fn(batch.num_graphs, batch.device), level="system")

    @staticmethod
    def all_complete(batch: Batch, exit_status: int) -> bool:
        status = _flat_status(batch)
        return status is not None and bool((status >= exit_status).all())

    def refill_check(self, batch: Batch, exit_status: int) -> Batch | None:
        """Move graduated systems (``status >= exit_status``) to the sinks and ask the sampler for
        replacements within the freed atom/edge/count budget.  Returns ``None`` when nothing is left."""
        if self.sampler is None:
            raise RuntimeError("refill_check requires a sampler to be configured.")
        status = _flat_status(batch)
        graduated = status >= exit_status
        if not bool(graduated.any()):
            return batch
        remaining = torch.where(~graduated)[0]
        if self.sinks:
            self._overflow_to_sinks(batch, mask=graduated)
        n_rem = int(remaining.numel())
        result = batch.index_select(remaining) if n_rem else None
        s = self.sampler
        rem_atoms = result.num_nodes if result is not None else 0
        rem_edges = result.num_edges if result is not None else 0
        repl = s.request_replacements_budget(
            atom_budget=None if s.max_atoms is None else s.max_atoms - rem_atoms,
            edge_budget=None if s.max_edges is None else s.max_edges - rem_edges,
            max_count=None if s.max_batch_size is None else s.max_batch_size - n_rem)
        n_new = len(repl)
        if n_new:
            new_batch = Batch.from_data_list(repl, device=batch.device)
            self._ensure_bookkeeping_fields(new_batch)
            if result is None:
                result = new_batch
            else:
                for key in list(result._storage.keys()):
                    if key not in new_batch:
                        ref = result[key]
                        lvl = result._storage.group_of(key)
                        rows = {"atoms": new_batch.num_nodes, "edges": new_batch.num_edges,
                                "system": new_batch.num_graphs}[lvl]
                        if lvl == "edges" and new_batch._edges_group is None:
                            continue
                        new_batch.add_key(key, ref.new_zeros((rows,) + tuple(ref.shape[1:])),
                                          level={"atoms": "node", "edges": "edge", "system": "system"}[lvl])
                result.append(new_batch)
        if result is not None:
            self._sync_state_to_batch(remaining, n_new, result)
            return result
        if s.exhausted:
            self.done = True
        self._state = None
        return None

    # ---- composition -----------------------------------------------------------
    def __add__(self, other: "BaseDynamics") -> "FusedStage":
        if isinstance(self, FusedStage):
            subs = list(self.sub_stages) + [(len(self.sub_stages), other)]
        else:
            subs = [(0, self), (1, other)]
        return FusedStage(sub_stages=subs, sampler=self.sampler or other.sampler, sinks=self.sinks or other.sinks,
                          refill_frequency=self.refill_frequency, device_type=self.device_type)

    def __or__(self, other: "BaseDynamics") -> Any:
        from nvalchemi_toolkit_b200.dynamics.pipeline import DistributedPipeline

        if isinstance(other, DistributedPipeline):
            stages = {0: self, **{r + 1: st for r, st in other.stages.items()}}
            return DistributedPipeline(stages=stages)
        return DistributedPipeline(stages={0: self, 1: other})


class FusedStage(BaseDynamics):
    """Several dynamics sharing one batch and one model evaluation per step."""

    def __init__(self, sub_stages: list[tuple[int, BaseDynamics]], *, entry_status: int = 0, exit_status: int = -1,
                 compile_step: bool = False, compile_kwargs: dict | None = None,
                 init_fn: Callable[[Batch], None] | None = None, **kwargs: Any) -> None:
        first = sub_stages[0][1]
        kinds = {d.device_type for _, d in sub_stages}
        if len(kinds) > 1:
            raise ValueError("All sub-stages in a FusedStage must share the same device_type, but got: "
                             f"{ {c: d.device_type for c, d in sub_stages} }.")
        kwargs.setdefault("device_type", first.device_type)
        super().__init__(model=first.model, **kwargs)
        self.sub_stages = list(sub_stages)
        self.__needs_keys__ = set().union(*(d.__needs_keys__ for _, d in sub_stages))
        self.__provides_keys__ = set().union(*(d.__provides_keys__ for _, d in sub_stages))
        self.entry_status = entry_status
        self.exit_status = len(sub_stages) if exit_status == -1 else exit_status
        self.compile_step, self.compile_kwargs = compile_step, dict(compile_kwargs or {})
        self.convergence_check_frequency = 1
        self.init_fn = init_fn
        self.fused_hooks: list = []
        for i, (code, dyn) in enumerate(self.sub_stages):
            if i + 1 < len(self.sub_stages):
                target = self.sub_stages[i + 1][0]
            elif dyn.convergence_hook is not None:
                target = self.exit_status
            else:
                continue
            dyn.hooks = [h for h in dyn.hooks if not (isinstance(h, ConvergenceHook) and h.source_status == code
                                                      and h.target_status == target)]
            if dyn.convergence_hook is not None:
                dyn.register_hook(ConvergenceHook(criteria=dyn.convergence_hook.criteria, source_status=code,
                                                  target_status=target))
            if dyn.n_steps is not None:
                BaseDynamics.register_bookkeeping_key(
                    f"n_steps_counter_{code}", lambda n, dev: torch.zeros(n, 1, dtype=torch.long, device=dev))

    def compile(self, **kwargs: Any) -> "FusedStage":
        """Accepted for API compatibility and reported as a no-op: the step already runs precompiled hand-written
        kernels and nothing here goes through a tracing compiler."""
        import warnings

        warnings.warn("FusedStage.compile() has no effect in this package: the fused step runs precompiled kernels",
                      UserWarning, stacklevel=2)
        return self

    def register_fused_hook(self, hook: Any) -> None:
        self.fused_hooks.append(hook)

    def _call_fused_hooks(self, stage: DynamicsStage, batch: Batch) -> None:
        ctx = None
        for h in self.fused_hooks:
            if (getattr(h, "_runs_on_stage", None) and h._runs_on_stage(stage)) or h.stage == stage:
                if self.step_count % h.frequency == 0:
                    ctx = ctx or self._build_context(batch)
                    h(ctx, stage)

    def _init_state(self, batch: Batch) -> None:
        for _, d in self.sub_stages:
            d._init_state(batch)

    def _ensure_state_initialized(self, batch: Batch) -> None:
        for _, d in self.sub_stages:
            d._ensure_state_initialized(batch)

    def _sync_state_to_batch(self, remaining_indices: torch.Tensor, n_new: int, template_batch: Batch) -> None:
        for _, d in self.sub_stages:
            d._sync_state_to_batch(remaining_indices, n_new, template_batch)

    def step(self, batch: Batch) -> tuple[Batch, torch.Tensor | None]:
        return self._step_impl(batch)

    def _step_impl(self, batch: Batch) -> tuple[Batch, torch.Tensor | None]:
        S = DynamicsStage
        self._ensure_bookkeeping_fields(batch)
        self._ensure_state_initialized(batch)
        self._call_fused_hooks(S.BEFORE_STEP, batch)
        self._call_hooks(S.BEFORE_STEP, batch)
        for _, d in self.sub_stages:
            d._call_hooks(S.BEFORE_STEP, batch)
        status = _flat_status(batch)
        masks = []
        for code, d in self.sub_stages:
            mask = status == code
            masks.append(mask)
            d._call_hooks(S.BEFORE_PRE_UPDATE, batch)
            if bool(mask.any()):
                d._masked_pre_update(batch, mask)
            d._call_hooks(S.AFTER_PRE_UPDATE, batch)
        self._call_hooks(S.BEFORE_COMPUTE, batch)
        for _, d in self.sub_stages:
            d._call_hooks(S.BEFORE_COMPUTE, batch)
        outputs = self.compute(batch)
        for k, v in outputs.items():
            if k not in ("forces", "energy") and isinstance(v, torch.Tensor) and k not in self._OUTPUT_KEY_TO_BATCH_ATTR:
                try:
                    batch[k] = v
                except (KeyError, ValueError):
                    pass
        self._call_hooks(S.AFTER_COMPUTE, batch)
        for _, d in self.sub_stages:
            d._call_hooks(S.AFTER_COMPUTE, batch)
        for (code, d), mask in zip(self.sub_stages, masks):
            d._call_hooks(S.BEFORE_POST_UPDATE, batch)
            if bool(mask.any()):
                d._masked_post_update(batch, mask)
            d._call_hooks(S.AFTER_POST_UPDATE, batch)
        pre_status = _flat_status(batch).clone()
        for _, d in self.sub_stages:
            d._call_hooks(S.AFTER_STEP, batch)  # per-stage ConvergenceHooks migrate status here
        self._call_hooks(S.AFTER_STEP, batch)
        self._call_fused_hooks(S.AFTER_STEP, batch)
        for i, (code, d) in enumerate(self.sub_stages):
            if d.n_steps is None:
                continue
            key = f"n_steps_counter_{code}"
            if getattr(batch, key, None) is None:
                batch.add_key(key, torch.zeros(batch.num_graphs, 1, dtype=torch.long, device=batch.device), "system")
            counter = getattr(batch, key).reshape(-1)
            cur = _flat_status(batch)
            active = cur == code
            counter += active.long()
            nxt = self.sub_stages[i + 1][0] if i + 1 < len(self.sub_stages) else self.exit_status
            migrate = active & (counter >= d.n_steps)
            cur.masked_fill_(migrate, nxt)
            counter.masked_fill_(migrate, 0)
        post_status = _flat_status(batch)
        for mask, (code, d) in zip(masks, self.sub_stages):
            moved = mask & (post_status != pre_status)
            d._last_converged = torch.where(moved)[0] if bool(moved.any()) else None
            if d._last_converged is not None:
                d._call_hooks(S.ON_CONVERGE, batch)
        self.step_count += 1
        for _, d in self.sub_stages:
            d.step_count += 1
        newly = (pre_status < self.exit_status) & (post_status >= self.exit_status)
        return batch, (torch.where(newly)[0] if bool(newly.any()) else None)

    def run(self, batch: Batch | None = None, n_steps: int | None = None) -> Batch | None:
        if batch is None:
            if self.sampler is None:
                raise ValueError("No batch provided and no sampler configured.")
            batch = self.sampler.build_initial_batch()
            if batch.device.type != self.device_type:  # datasets live on the host; the workflow runs on its device
                batch = batch.to(self.device)
            if self.init_fn is not None:
                self.init_fn(batch)
            self.active_batch = batch
        self._ensure_bookkeeping_fields(batch)
        resolved = n_steps if n_steps is not None else self.n_steps
        self._open_hooks()
        try:
            self._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
            for _, d in self.sub_stages:
                d._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
            self.compute(batch)
            self._call_hooks(DynamicsStage.AFTER_COMPUTE, batch)
            step_num = 0
            while True:
                batch, _ = self.step(batch)
                if self.sampler is not None and (step_num + 1) % self.refill_frequency == 0:
                    result = self.refill_check(batch, self.exit_status)
                    if result is None:
                        self.active_batch = None
                        return None
                    if result is not batch:
                        batch = result
                        self._last_converged = None  # system indices changed with the refill
                        for _, d in self.sub_stages:
                            d._last_converged = None
                        # forces of replacement systems are unknown: evaluate before the next pre_update
                        self._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
                        for _, d in self.sub_stages:
                            d._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)
                        self.compute(batch)
                    self.active_batch = batch
                elif self.sampler is None and (step_num + 1) % self.convergence_check_frequency == 0 \
                        and self.all_complete(batch, self.exit_status):
                    break
                step_num += 1
                if resolved is not None and step_num >= resolved:
                    break
            return batch
        finally:
            self._close_hooks()
