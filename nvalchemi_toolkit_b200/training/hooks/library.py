# SPDX-License-Identifier: Apache-2.0
"""Training hooks: data parallelism, update policies, AMP, EMA, checkpoints, fine-tuning patches.

Reference: ``nvalchemi/training/hooks/{ddp,update,mixed_precision,ema,checkpoint,finetune}.py``.  Update policies run in
priority order (accumulation 10 < AMP 20 < clipping 30 < loss-spike skip 40) and may veto the optimiser step by setting
``ctx.skip_optimizer_step``.  ``FusedGradAllReduceHook`` is this package's alternative to DDP on NVLink machines: one
kernel sums every rank's flat gradient buffer through peer memory and applies the ``1/world`` (and loss-scale) factor in
the same pass."""
from __future__ import annotations

import copy
import re
import threading
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Mapping

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.training._stages import TrainingStage as S
from nvalchemi_toolkit_b200.training.distributed import get_rank, get_world_size, init_distributed


class _Base:
    frequency = 1
    stage: Enum | None = None
    priority = 0


class TrainingUpdateHook(_Base):
    """Base of the hooks that shape ONE optimiser update: gradient accumulation, mixed precision, clipping, skipping of
    loss spikes (reference ``training/hooks/update.py:197-340``).

    They follow the plain hook protocol (``__call__(ctx, stage)``) and talk to the strategy and to each other through
    the training context instead of return values: ``ctx.loss`` may be replaced before the backward pass (scaling),
    ``ctx.accumulating = True`` keeps the previous gradients, ``ctx.skip_optimizer_step = True`` vetoes the optimiser and
    scheduler step of this batch (any hook may set it; later hooks read it and skip work that assumes a step, e.g.
    clipping), ``ctx.sync_gradients`` says whether this micro-batch ends with a step.  ``priority`` orders hooks that
    share a stage, lower first: 10 accumulation, 20 mixed precision, 30 clipping, 40 spike skipping, default 50.
    ``a + b`` builds a :class:`TrainingUpdateOrchestrator` that dispatches them in that order."""

    priority = 50

    def __add__(self, other: Any) -> "TrainingUpdateOrchestrator":
        mine = self.hooks if isinstance(self, TrainingUpdateOrchestrator) else [self]
        theirs = other.hooks if isinstance(other, TrainingUpdateOrchestrator) else [other]
        return TrainingUpdateOrchestrator(list(mine) + list(theirs))


# ------------------------------------------------------------------ data parallel
class DDPHook(_Base):
    """Wraps the configured models in ``DistributedDataParallel`` at SETUP and shards the dataloader."""

    def __init__(self, model_keys: list[str] | None = None, find_unused_parameters: bool = False,
                 broadcast_buffers: bool = True, static_graph: bool = False, process_group: Any = None,
                 backend: str | None = None, auto_init: bool = True, sampler_cls: Any = None,
                 sampler_kwargs: dict | None = None, frequency: int = 1, stage: Enum = S.SETUP) -> None:
        self.model_keys, self.find_unused_parameters = model_keys, find_unused_parameters
        self.broadcast_buffers, self.static_graph = broadcast_buffers, static_graph
        self.process_group, self.backend, self.auto_init = process_group, backend, auto_init
        self.sampler_cls = sampler_cls or torch.utils.data.distributed.DistributedSampler
        self.sampler_kwargs = dict(sampler_kwargs or {})
        self.frequency, self.stage = frequency, stage

    def prepare_strategy(self, strategy: Any) -> None:
        if self.auto_init and not dist.is_initialized():
            init_distributed(self.backend)
        if torch.cuda.is_available() and strategy.devices[0].type == "cuda":
            import os

            strategy.devices = [torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))]

    def __call__(self, ctx: Any, stage: Enum) -> None:
        strategy = ctx.workflow
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return
        keys = self.model_keys or [k for k in strategy.models if k in strategy.optimizer_configs]
        for k in keys:
            m = strategy.models[k]
            if isinstance(m, torch.nn.parallel.DistributedDataParallel):
                continue
            dev = strategy.devices[0]
            strategy.models[k] = torch.nn.parallel.DistributedDataParallel(
                m, device_ids=[dev.index] if dev.type == "cuda" else None, process_group=self.process_group,
                find_unused_parameters=self.find_unused_parameters, broadcast_buffers=self.broadcast_buffers,
                static_graph=self.static_graph)
        strategy.active_dataloader = self.prepare_dataloader(strategy.active_dataloader)

    def prepare_dataloader(self, loader: Any) -> Any:
        if loader is None:
            return None
        if hasattr(loader, "set_distributed"):
            loader.set_distributed(dist.get_rank(), dist.get_world_size())
            return loader
        if isinstance(loader, torch.utils.data.DataLoader) and not isinstance(loader.sampler, self.sampler_cls):
            sampler = self.sampler_cls(loader.dataset, **self.sampler_kwargs)
            return torch.utils.data.DataLoader(loader.dataset, batch_size=loader.batch_size, sampler=sampler,
                                               num_workers=loader.num_workers, collate_fn=loader.collate_fn,
                                               pin_memory=loader.pin_memory, drop_last=loader.drop_last)
        return loader


class FusedGradAllReduceHook(_Base):
    """Gradient all-reduce over peer memory, bucketed and overlapped with the backward pass, with the ``1/world`` and
    loss-scale factors applied inside the reduction kernel.

    Parameters are packed (in reverse registration order, the order in which backward produces their gradients) into
    buckets of about ``bucket_mb`` MiB that live in a symmetric (peer-mapped) arena.  A
    ``register_post_accumulate_grad_hook`` on every parameter copies its finished gradient into its bucket; as soon as a
    bucket is complete (and all earlier buckets have been launched, so every rank issues the same sequence) its
    reduction is enqueued on a side stream: flag barrier, then one kernel that sums the peers' buckets (in the NVSwitch
    with ``multimem.ld_reduce`` when a multicast mapping exists, by peer loads otherwise) and scales, then a second
    barrier, while the main stream continues with the rest of backward.  ``AFTER_BACKWARD`` flushes what is left
    (parameters without a gradient contribute zeros and still receive the peers' sum), joins the side stream and
    writes the reduced values back into ``p.grad``.  Replaces PyTorch DDP's bucketed NCCL all-reduce
    (reference ``nvalchemi/training/hooks/ddp.py:250-301``).  Without CUDA peer memory (CPU / gloo) one
    ``torch.distributed`` all-reduce of the flat buffer is used, so the hook is testable on CPU ranks."""

    stage = S.AFTER_BACKWARD
    priority = 5

    def __init__(self, model_keys: list[str] | None = None, loss_scale: float = 1.0, frequency: int = 1,
                 status_check: str | None = "lazy", bucket_mb: float = 4.0, overlap: bool = True) -> None:
        self.model_keys, self.loss_scale, self.frequency = model_keys, loss_scale, frequency
        #: how a peer that missed the device-side rendezvous surfaces: "sync" (host read every step, raises before the
        #: gradients are used), "lazy" (raises at the next step, no host synchronisation) or None
        self.status_check = status_check
        self.bucket_mb, self.overlap = float(bucket_mb), bool(overlap)
        self._p2p = None
        self._flat = self._out = None
        self._params: list[torch.nn.Parameter] = []
        self._slots: dict[int, tuple[int, int, int]] = {}   # id(param) -> (bucket, offset, numel)
        self._buckets: list[dict] = []
        self._armed = False
        self._comm_stream: Any = None
        self.num_overlapped = 0  # buckets launched from inside backward during the last step

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in (S.BEFORE_BACKWARD, S.AFTER_BACKWARD)

    def prepare_strategy(self, strategy: Any) -> None:
        if not dist.is_initialized():
            init_distributed(None)

    def _setup(self, strategy: Any) -> None:
        keys = self.model_keys or [k for k in strategy.models if k in strategy.optimizer_configs]
        self._params = [p for k in keys for p in strategy.models[k].parameters() if p.requires_grad]
        dev = strategy.devices[0]
        for p in self._params:  # identical initial weights on every rank
            dist.broadcast(p.data, src=0)
        limit = max(1, int(self.bucket_mb * (1 << 20) / 4))
        off, cur = 0, {"start": 0, "numel": 0, "params": []}
        for p in reversed(self._params):
            if cur["params"] and cur["numel"] + p.numel() > limit:
                cur["numel"] = (cur["numel"] + 3) // 4 * 4  # 16-byte groups for the vector / multimem paths
                self._buckets.append(cur)
                off = cur["start"] + cur["numel"]
                cur = {"start": off, "numel": 0, "params": []}
            self._slots[id(p)] = (len(self._buckets), cur["start"] + cur["numel"], p.numel())
            cur["params"].append(p)
            cur["numel"] += p.numel()
        cur["numel"] = (cur["numel"] + 3) // 4 * 4
        self._buckets.append(cur)
        n = cur["start"] + cur["numel"]
        peer = dev.type == "cuda" and dist.get_backend() == "nccl"
        if peer:
            from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

            self._p2p = P2PContext(4 * n + 4096, dev)
            self._flat, _ = self._p2p.arena.alloc((n,), torch.float32)
            self._out = torch.empty(n, dtype=torch.float32, device=dev)
            self._comm_stream = torch.cuda.Stream(device=dev)
            base = self._p2p.arena.offset_of(self._flat)
            for b in self._buckets:
                b["ptrs"] = torch.tensor([a + base + 4 * b["start"] for a in self._p2p.arena.base_ptrs], dtype=torch.int64,
                                         device=dev)
        else:
            self._flat = torch.zeros(n, dtype=torch.float32, device=dev)
        for b in self._buckets:
            b["ready"], b["launched"] = 0, False
        if peer and self.overlap:
            for p in self._params:
                p.register_post_accumulate_grad_hook(self._on_grad)

    # ---- overlap with backward ------------------------------------------------------------------------------------
    def _on_grad(self, p: torch.nn.Parameter) -> None:
        if not self._armed:
            return
        bi, off, n = self._slots[id(p)]
        self._flat[off: off + n].copy_(p.grad.reshape(-1))
        b = self._buckets[bi]
        b["ready"] += 1
        self._launch_ready(count=True)

    def _launch_ready(self, count: bool = False) -> None:
        """Enqueue, in bucket order, every bucket whose gradients are all in place."""
        for b in self._buckets:
            if b["launched"]:
                continue
            if b["ready"] < len(b["params"]):
                break
            self._launch(b)
            if count:
                self.num_overlapped += 1

    def _launch(self, b: dict) -> None:
        world = dist.get_world_size()
        scale = 1.0 / (world * self.loss_scale)
        view = self._flat[b["start"]: b["start"] + b["numel"]]
        out = self._out[b["start"]: b["start"] + b["numel"]]
        done = torch.cuda.Event()
        done.record()  # the copies into this bucket (current stream) precede the reduction
        self._comm_stream.wait_event(done)
        with torch.cuda.stream(self._comm_stream):
            b["result"] = self._p2p.allreduce_(view, scale, out=out, check=None, ptrs=b["ptrs"])
        b["launched"] = True

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return
        if self._flat is None:
            self._setup(ctx.workflow)
        if stage == S.BEFORE_BACKWARD:
            self._armed = self._p2p is not None and self.overlap and getattr(ctx, "sync_gradients", True)
            self.num_overlapped = 0
            for b in self._buckets:
                b["ready"], b["launched"] = 0, False
            if self._p2p is not None and self.status_check == "lazy":
                self._p2p.check(wait=False)  # a rendezvous missed in the previous step surfaces here
            return
        if not getattr(ctx, "sync_gradients", True):
            return  # gradients keep accumulating locally; the reduction happens with the last micro-batch
        world = dist.get_world_size()
        armed, self._armed = self._armed, False
        if self._p2p is not None:
            for p in self._params:
                bi, off, n = self._slots[id(p)]
                b = self._buckets[bi]
                if armed and b["launched"]:
                    continue
                if p.grad is None:
                    self._flat[off: off + n].zero_()
                elif not armed or b["ready"] < len(b["params"]):
                    self._flat[off: off + n].copy_(p.grad.reshape(-1))
            for b in self._buckets:
                if not b["launched"]:
                    b["ready"] = len(b["params"])
            self._launch_ready()
            torch.cuda.current_stream().wait_stream(self._comm_stream)
            if self.status_check == "sync":
                self._p2p.check(wait=True)
            elif self.status_check == "lazy":
                self._p2p.post_status()
            result = None
        else:
            for p in self._params:
                _, off, n = self._slots[id(p)]
                if p.grad is None:
                    self._flat[off: off + n].zero_()
                else:
                    self._flat[off: off + n].copy_(p.grad.reshape(-1))
            dist.all_reduce(self._flat)
            result = self._flat.mul_(1.0 / (world * self.loss_scale))
        for p in self._params:
            bi, off, n = self._slots[id(p)]
            if result is not None:
                src = result[off: off + n]
            else:
                b = self._buckets[bi]
                src = b["result"][off - b["start"]: off - b["start"] + n]
            if p.grad is None:
                # a parameter unused on this rank still receives the peers' contribution: every rank must apply the
                # same reduced gradient or the replicas drift apart
                p.grad = torch.empty_like(p)
            p.grad.copy_(src.reshape(p.shape))


# ------------------------------------------------------------------ update policies
class GradientAccumulationHook(TrainingUpdateHook):
    """Steps the optimiser every ``steps`` batches; gradients accumulate in between (loss scaled by ``1/steps``)."""

    priority = 10

    def __init__(self, steps: int = 1) -> None:
        self.steps = steps

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in (S.BEFORE_BATCH, S.AFTER_LOSS, S.BEFORE_OPTIMIZER_STEP)

    def __call__(self, ctx: Any, stage: Enum) -> None:
        k = ctx.batch_count % self.steps
        if stage == S.BEFORE_BATCH:
            ctx.accumulating = k != 0                     # keep the gradients of the previous micro-batches
            ctx.sync_gradients = k == self.steps - 1      # the micro-batch that ends with the optimiser step
        elif stage == S.AFTER_LOSS and self.steps > 1:
            ctx.loss = ctx.loss / self.steps
        elif stage == S.BEFORE_OPTIMIZER_STEP and k != self.steps - 1:
            ctx.skip_optimizer_step = True


class MixedPrecisionHook(TrainingUpdateHook):
    """Autocast around forward + loss, scaled backward, ``GradScaler`` step (claims both DO slots)."""

    priority = 20

    def __init__(self, dtype: torch.dtype = torch.bfloat16, enabled: bool = True, use_grad_scaler: bool | None = None,
                 device_type: str | None = None) -> None:
        self.dtype, self.enabled = dtype, enabled
        self.device_type = device_type or ("cuda" if torch.cuda.is_available() else "cpu")
        use = (dtype == torch.float16) if use_grad_scaler is None else use_grad_scaler
        self.scaler = torch.amp.GradScaler(self.device_type, enabled=use and enabled)
        self._cm: Any = None

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in (S.BEFORE_FORWARD, S.AFTER_LOSS, S.DO_BACKWARD, S.BEFORE_OPTIMIZER_STEP, S.DO_OPTIMIZER_STEP)

    def __call__(self, ctx: Any, stage: Enum) -> None:
        if stage == S.BEFORE_FORWARD:
            self._cm = torch.autocast(self.device_type, dtype=self.dtype, enabled=self.enabled)
            self._cm.__enter__()
        elif stage == S.AFTER_LOSS:
            if self._cm is not None:
                self._cm.__exit__(None, None, None)
                self._cm = None
            ctx.grad_scaler = self.scaler
        elif stage == S.DO_BACKWARD:
            self.scaler.scale(ctx.loss).backward()
        elif stage == S.BEFORE_OPTIMIZER_STEP:
            for o in ctx.optimizers:
                self.scaler.unscale_(o)
        elif stage == S.DO_OPTIMIZER_STEP:
            for o in ctx.optimizers:
                self.scaler.step(o)
            self.scaler.update()

    def state_dict(self) -> Mapping[str, Any]:
        return {"scaler": self.scaler.state_dict()}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        self.scaler.load_state_dict(state["scaler"])


class GradientClipHook(TrainingUpdateHook):
    stage = S.BEFORE_OPTIMIZER_STEP
    priority = 30

    def __init__(self, max_norm: float = 10.0, norm_type: float = 2.0) -> None:
        self.max_norm, self.norm_type = max_norm, norm_type
        self.last_norm: float | None = None

    def __call__(self, ctx: Any, stage: Enum) -> None:
        params = [p for o in ctx.optimizers for g in o.param_groups for p in g["params"] if p.grad is not None]
        if params:
            self.last_norm = float(torch.nn.utils.clip_grad_norm_(params, self.max_norm, self.norm_type))


class LossSpikeSkipHook(TrainingUpdateHook):
    """Skips the update when the loss exceeds ``factor`` x its running mean (or is not finite)."""

    stage = S.BEFORE_OPTIMIZER_STEP
    priority = 40

    def __init__(self, factor: float = 10.0, momentum: float = 0.98, warmup: int = 20) -> None:
        self.factor, self.momentum, self.warmup = factor, momentum, warmup
        self.mean: float | None = None
        self.seen = 0
        self.skipped = 0

    def __call__(self, ctx: Any, stage: Enum) -> None:
        loss = float(ctx.loss.detach())
        bad = not (loss == loss and abs(loss) != float("inf"))
        if not bad and self.mean is not None and self.seen >= self.warmup and loss > self.factor * self.mean:
            bad = True
        if bad:
            ctx.skip_optimizer_step = True
            self.skipped += 1
            return
        self.mean = loss if self.mean is None else self.momentum * self.mean + (1 - self.momentum) * loss
        self.seen += 1

    def state_dict(self) -> Mapping[str, Any]:
        return {"mean": self.mean, "seen": self.seen, "skipped": self.skipped}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        self.mean, self.seen, self.skipped = state["mean"], state["seen"], state["skipped"]


class TrainingUpdateOrchestrator(TrainingUpdateHook):
    """Runs a set of update hooks in priority order at each stage they subscribe to (priority-ordered veto chain)."""

    def __init__(self, hooks: list[Any]) -> None:
        self.hooks = sorted(hooks, key=lambda h: getattr(h, "priority", 0))

    def _runs_on_stage(self, stage: Enum) -> bool:
        return any(self._sub(h, stage) for h in self.hooks)

    @staticmethod
    def _sub(h: Any, stage: Enum) -> bool:
        r = getattr(h, "_runs_on_stage", None)
        return bool(r(stage)) if r is not None else h.stage == stage

    def __call__(self, ctx: Any, stage: Enum) -> None:
        for h in self.hooks:
            if self._sub(h, stage):
                h(ctx, stage)

    def state_dict(self) -> Mapping[str, Any]:
        return {type(h).__name__: dict(h.state_dict()) for h in self.hooks if hasattr(h, "state_dict")}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        for h in self.hooks:
            if hasattr(h, "load_state_dict") and type(h).__name__ in state:
                h.load_state_dict(state[type(h).__name__])


# ------------------------------------------------------------------ EMA, checkpoints
class EMAHook(_Base):
    """Exponential moving average of a model's parameters, updated after every optimiser step (checkpointable)."""

    stage = S.AFTER_OPTIMIZER_STEP
    checkpoint_name = "EMAHook"

    def __init__(self, model_key: str = "main", decay: float = 0.999, use_as_inference_model: bool = True,
                 frequency: int = 1) -> None:
        self.model_key, self.decay, self.use_as_inference_model, self.frequency = model_key, decay, use_as_inference_model, frequency
        self.ema: torch.nn.Module | None = None
        self.num_updates = 0

    def _ensure(self, strategy: Any) -> None:
        if self.ema is None:
            src = strategy.models[self.model_key]
            src = src.module if isinstance(src, torch.nn.parallel.DistributedDataParallel) else src
            self.ema = copy.deepcopy(src).eval()
            for p in self.ema.parameters():
                p.requires_grad_(False)
            if self.use_as_inference_model:
                strategy.inference_model = self.ema

    def __call__(self, ctx: Any, stage: Enum) -> None:
        self._ensure(ctx.workflow)
        src = ctx.workflow.models[self.model_key]
        src = src.module if isinstance(src, torch.nn.parallel.DistributedDataParallel) else src
        self.num_updates += 1
        d = min(self.decay, (1 + self.num_updates) / (10 + self.num_updates))
        with torch.no_grad():
            for pe, ps in zip(self.ema.parameters(), src.parameters()):
                pe.mul_(d).add_(ps.detach(), alpha=1 - d)
            for be, bs in zip(self.ema.buffers(), src.buffers()):
                be.copy_(bs)

    def state_dict(self) -> Mapping[str, Any]:
        return {"num_updates": self.num_updates, "ema": None if self.ema is None else self.ema.state_dict()}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        self.num_updates = state["num_updates"]
        self._pending = state["ema"]
        if self.ema is not None and state["ema"] is not None:
            self.ema.load_state_dict(state["ema"])


class CheckpointHook(_Base):
    """Saves a manifest checkpoint every ``every_n_steps`` optimiser steps and/or ``every_n_epochs`` epochs."""

    def __init__(self, directory: str | Path, every_n_steps: int | None = None, every_n_epochs: int | None = 1,
                 asynchronous: bool = False, rank_zero_only: bool = True) -> None:
        self.directory, self.every_n_steps, self.every_n_epochs = Path(directory), every_n_steps, every_n_epochs
        self.asynchronous, self.rank_zero_only = asynchronous, rank_zero_only
        self._pending: Any = None
        self._last_step = -1

    def _runs_on_stage(self, stage: Enum) -> bool:
        return stage in (S.AFTER_BATCH, S.AFTER_EPOCH, S.AFTER_TRAINING)

    def __call__(self, ctx: Any, stage: Enum) -> None:
        st = ctx.workflow
        due = (stage == S.AFTER_BATCH and self.every_n_steps and st.step_count and st.step_count % self.every_n_steps == 0
               and st.step_count != self._last_step) or \
              (stage == S.AFTER_EPOCH and self.every_n_epochs and st.epoch_count % self.every_n_epochs == 0) or \
              (stage == S.AFTER_TRAINING and st.step_count != self._last_step)
        if not due or (self.rank_zero_only and get_rank(st.distributed_manager) != 0):
            return
        self._last_step = st.step_count
        if self._pending is not None:  # one writer at a time: the previous files are complete before the next index
            self._pending.wait()
            self._pending = None
        if self.asynchronous and stage != S.AFTER_TRAINING:
            # states are snapshotted to pinned host memory here; the files are written while training goes on
            out = st.save_checkpoint(self.directory, asynchronous=True)
            self._pending = out if hasattr(out, "wait") else None
        else:
            st.save_checkpoint(self.directory)


# ------------------------------------------------------------------ fine-tuning helpers
class ModulePatchHook(_Base):
    """Replaces sub-modules (by dotted name) at SETUP, e.g. a fresh readout head for fine-tuning."""

    stage = S.SETUP

    def __init__(self, patches: dict[str, Callable[[torch.nn.Module], torch.nn.Module]], model_key: str = "main") -> None:
        self.patches, self.model_key = patches, model_key

    def __call__(self, ctx: Any, stage: Enum) -> None:
        root = ctx.workflow.models[self.model_key]
        for name, factory in self.patches.items():
            parent = root
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], factory(getattr(parent, parts[-1])))


class TrainableParameterHook(_Base):
    """Freezes every parameter whose name does not match one of the regular expressions."""

    stage = S.SETUP

    def __init__(self, trainable: list[str], model_key: str = "main") -> None:
        self.patterns, self.model_key = [re.compile(p) for p in trainable], model_key
        self.num_trainable = 0

    def __call__(self, ctx: Any, stage: Enum) -> None:
        self.num_trainable = 0
        for n, p in ctx.workflow.models[self.model_key].named_parameters():
            on = any(r.search(n) for r in self.patterns)
            p.requires_grad_(on)
            self.num_trainable += int(on) * p.numel()
