# SPDX-License-Identifier: Apache-2.0
"""``TrainingStrategy``: the hook-driven training loop.

Follows the reference's loop (``nvalchemi/training/strategy.py:946-997,1189-1302``): per batch
``BEFORE_BATCH → zero_grad → BEFORE_FORWARD → training_fn → AFTER_FORWARD → BEFORE_LOSS → loss → AFTER_LOSS →
BEFORE_BACKWARD → backward (or the DO_BACKWARD claimant) → AFTER_BACKWARD → BEFORE_OPTIMIZER_STEP → step (or the
DO_OPTIMIZER_STEP claimant) → AFTER_OPTIMIZER_STEP → AFTER_BATCH``; counters ``step_count, global_step_count,
batch_count, epoch_count, epoch_step_count`` survive checkpoints so a resumed run continues mid-epoch regardless of the
world size.  ``ctx.skip_optimizer_step`` lets update hooks (accumulation, loss-spike skip, AMP overflow) veto a step.
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Callable, Iterable

import torch

from nvalchemi_toolkit_b200._serialization import import_from_path, type_to_path
from nvalchemi_toolkit_b200.hooks.core import HookRegistryMixin, TrainContext
from nvalchemi_toolkit_b200.training import checkpoint as ckpt
from nvalchemi_toolkit_b200.training._stages import TrainingStage
from nvalchemi_toolkit_b200.training.distributed import get_rank, get_world_size
from nvalchemi_toolkit_b200.training.losses import BaseLossFunction, ComposedLossFunction
from nvalchemi_toolkit_b200.training.optimizers import OptimizerConfig, setup_optimizers, step_schedulers, zero_gradients


def default_training_fn(model: Any, batch: Any) -> dict[str, torch.Tensor]:
    """Forward of a ``BaseModelMixin`` wrapper in training mode; returns its canonical outputs."""
    return model(batch)


class TrainingStrategy(HookRegistryMixin):
    _stage_type = TrainingStage

    def __init__(self, models: "dict[str, torch.nn.Module] | torch.nn.Module", optimizer_configs: Any = None,
                 loss_fn: Any = None, num_epochs: int | None = None, num_steps: int | None = None,
                 training_fn: "Callable | str | None" = None, devices: list | None = None, hooks: list | None = None,
                 validation_config: Any = None, inference_model: Any = None, distributed_manager: Any = None) -> None:
        if isinstance(models, torch.nn.Module):
            models = {"main": models}
        self.models: dict[str, torch.nn.Module] = dict(models)
        if optimizer_configs is None:
            optimizer_configs = {"main": [OptimizerConfig()]}
        if isinstance(optimizer_configs, OptimizerConfig):
            optimizer_configs = {"main": [optimizer_configs]}
        self.optimizer_configs = {k: (v if isinstance(v, (list, tuple)) else [v]) for k, v in optimizer_configs.items()}
        if isinstance(loss_fn, BaseLossFunction):
            loss_fn = ComposedLossFunction([loss_fn])
        self.loss_fn = loss_fn
        if (num_epochs is None) == (num_steps is None):
            raise ValueError("exactly one of num_epochs / num_steps must be given")
        self.num_epochs, self.num_steps = num_epochs, num_steps
        if isinstance(training_fn, str):
            training_fn = import_from_path(training_fn)
        self.training_fn = training_fn or default_training_fn
        self.devices = [torch.device(d) for d in (devices or ["cuda" if torch.cuda.is_available() else "cpu"])]
        self.validation_config = validation_config
        self.inference_model = inference_model
        self.distributed_manager = distributed_manager
        self.step_count = self.global_step_count = self.batch_count = self.epoch_count = self.epoch_step_count = 0
        self.last_validation: dict[str, Any] | None = None
        self.last_losses: dict[str, torch.Tensor] | None = None
        self._optimizers: list = []
        self._lr_schedulers: list = []
        self._opt_cfgs: list[OptimizerConfig] = []
        self._ctx: TrainContext | None = None
        self._setup_done = False
        self.active_dataloader: Any = None
        self.optimizer_parameter_filter: set[str] | None = None
        self._init_hooks(hooks)

    # ---- properties / hooks ---------------------------------------------------------
    @property
    def single_model_input(self) -> bool:
        return set(self.models) == {"main"}

    @property
    def epoch(self) -> int:
        return self.epoch_count

    def register_hook(self, hook: Any, stage: Any = None) -> None:
        super().register_hook(hook, stage)
        for claim in (TrainingStage.DO_BACKWARD, TrainingStage.DO_OPTIMIZER_STEP):
            n = sum(1 for h in self.hooks if self._subscribes(h, claim))
            if n > 1:
                raise ValueError(f"more than one hook claims {claim.name}")

    @staticmethod
    def _subscribes(hook: Any, stage: TrainingStage) -> bool:
        runs = getattr(hook, "_runs_on_stage", None)
        return bool(runs(stage)) if runs is not None else hook.stage == stage

    def _claimed(self, stage: TrainingStage) -> bool:
        return any(self._subscribes(h, stage) for h in self.hooks)

    def _build_context(self, batch: Any) -> TrainContext:
        if self._ctx is not None:
            self._ctx.batch = batch
            return self._ctx
        ctx = TrainContext(batch=batch, model=self.models.get("main"), global_rank=get_rank(self.distributed_manager),
                           workflow=self, step_count=self.step_count, global_step_count=self.global_step_count,
                           batch_count=self.batch_count, epoch_step_count=self.epoch_step_count, epoch=self.epoch_count,
                           models=self.models, optimizers=self._optimizers, lr_schedulers=self._lr_schedulers,
                           validation=self.last_validation)
        ctx.skip_optimizer_step = False  # type: ignore[attr-defined]
        return ctx

    def _run_hooks(self, stage: TrainingStage, batch: Any) -> None:
        self._call_hooks(stage, batch)

    # ---- setup --------------------------------------------------------------------------
    def _setup(self, dataloader: Any = None) -> Any:
        if self._setup_done:
            return dataloader
        for h in self.hooks:
            prep = getattr(h, "prepare_strategy", None)
            if prep is not None:
                prep(self)
        dev = self.devices[0]
        for k, m in self.models.items():
            self.models[k] = m.to(dev)
        self.active_dataloader = dataloader
        self._run_hooks(TrainingStage.SETUP, None)
        dataloader = self.active_dataloader
        self._optimizers, self._lr_schedulers, self._opt_keys = setup_optimizers(self.models, self.optimizer_configs,
                                                                                 self.optimizer_parameter_filter)
        self._opt_cfgs = [c for k in self.optimizer_configs for c in self.optimizer_configs[k]]
        pending = getattr(self, "_pending_restore", None)
        if pending is not None:
            meta = ckpt.load_checkpoint(pending[0], self.models, self._optimizers, self._lr_schedulers, self.hooks,
                                        step=pending[1], map_location=dev, optimizer_keys=self._opt_keys)
            self._apply_meta(meta)
            self._pending_restore = None
        for k, m in self.models.items():
            if k in self.optimizer_configs:
                m.train()
            else:
                m.eval()
                for p in m.parameters():
                    p.requires_grad_(False)
        self._setup_done = True
        return dataloader

    # ---- one batch ----------------------------------------------------------------------------
    def train_batch(self, batch: Any) -> dict[str, torch.Tensor]:
        self._setup()
        batch = batch.to(self.devices[0], non_blocking=True) if hasattr(batch, "to") else batch
        self._ctx = None
        self._ctx = self._build_context(batch)
        ctx = self._ctx
        try:
            self._run_hooks(TrainingStage.BEFORE_BATCH, batch)
            if not getattr(ctx, "accumulating", False):
                zero_gradients(self._optimizers)
            self._run_hooks(TrainingStage.BEFORE_FORWARD, batch)
            model_arg = self.models["main"] if self.single_model_input else self.models
            predictions = self.training_fn(model_arg, batch)
            ctx.predictions = predictions
            self._run_hooks(TrainingStage.AFTER_FORWARD, batch)
            self._run_hooks(TrainingStage.BEFORE_LOSS, batch)
            losses = self.loss_fn(predictions, batch, step=self.step_count, epoch=self.epoch_count)
            ctx.loss, ctx.losses = losses["total_loss"], losses
            self.last_losses = {k: v.detach() for k, v in losses.items()}
            self._run_hooks(TrainingStage.AFTER_LOSS, batch)
            self._run_hooks(TrainingStage.BEFORE_BACKWARD, batch)
            if self._claimed(TrainingStage.DO_BACKWARD):
                self._run_hooks(TrainingStage.DO_BACKWARD, batch)
            else:
                ctx.loss.backward()
            self._run_hooks(TrainingStage.AFTER_BACKWARD, batch)
            self._run_hooks(TrainingStage.BEFORE_OPTIMIZER_STEP, batch)
            stepped = False
            if not getattr(ctx, "skip_optimizer_step", False):
                if self._claimed(TrainingStage.DO_OPTIMIZER_STEP):
                    self._run_hooks(TrainingStage.DO_OPTIMIZER_STEP, batch)
                    stepped = not getattr(ctx, "skip_optimizer_step", False)
                else:
                    for o in self._optimizers:
                        o.step()
                    stepped = True
                if stepped:
                    step_schedulers(self._lr_schedulers, self._opt_cfgs, "step")
                    self._run_hooks(TrainingStage.AFTER_OPTIMIZER_STEP, batch)
            self.batch_count += 1
            self.epoch_step_count += 1
            if stepped:
                self.step_count += 1
                self.global_step_count += get_world_size(self.distributed_manager)
            ctx.step_count, ctx.global_step_count = self.step_count, self.global_step_count
            ctx.batch_count, ctx.epoch_step_count = self.batch_count, self.epoch_step_count
            self._run_hooks(TrainingStage.AFTER_BATCH, batch)
            return self.last_losses
        finally:
            self._ctx = None

    # ---- full run -----------------------------------------------------------------------------------
    def _target_steps(self, per_epoch: int | None) -> int | None:
        if self.num_steps is not None:
            return self.num_steps
        return None if per_epoch is None else self.num_epochs * per_epoch

    def run(self, dataloader: Iterable, validation_dataloader: Iterable | None = None) -> "TrainingStrategy":
        dataloader = self._setup(dataloader)
        per_epoch = len(dataloader) if hasattr(dataloader, "__len__") else None
        self._run_hooks(TrainingStage.BEFORE_TRAINING, None)
        done = False
        while not done:
            if self.num_epochs is not None and self.epoch_count >= self.num_epochs:
                break
            for obj in (dataloader, getattr(dataloader, "sampler", None), getattr(dataloader, "batch_sampler", None)):
                if obj is not None and hasattr(obj, "set_epoch"):
                    obj.set_epoch(self.epoch_count)
            skip = self.epoch_step_count  # mid-epoch resume
            if skip and hasattr(dataloader, "set_epoch_step"):
                dataloader.set_epoch_step(skip)
                skip = 0
            self._run_hooks(TrainingStage.BEFORE_EPOCH, None)
            for i, batch in enumerate(dataloader):
                if i < skip:
                    continue
                self.train_batch(batch)
                self._maybe_validate(TrainingStage.AFTER_BATCH, validation_dataloader)
                if self.num_steps is not None and self.step_count >= self.num_steps:
                    done = True
                    break
            else:
                self.epoch_count += 1
                self.epoch_step_count = 0
                step_schedulers(self._lr_schedulers, self._opt_cfgs, "epoch")
                self._run_hooks(TrainingStage.AFTER_EPOCH, None)
                self._maybe_validate(TrainingStage.AFTER_EPOCH, validation_dataloader)
            if per_epoch == 0:
                break
        self._run_hooks(TrainingStage.AFTER_TRAINING, None)
        return self

    # ---- validation ---------------------------------------------------------------------------------------
    def _maybe_validate(self, stage: TrainingStage, loader: Iterable | None) -> None:
        cfg = self.validation_config
        if cfg is None:
            return
        loader = loader if loader is not None else cfg.data
        if loader is None:
            return
        due = (stage == TrainingStage.AFTER_BATCH and cfg.every_n_steps and self.step_count
               and self.step_count % cfg.every_n_steps == 0) or \
              (stage == TrainingStage.AFTER_EPOCH and cfg.every_n_epochs and self.epoch_count % cfg.every_n_epochs == 0)
        if due:
            self.validate(loader)

    def validate(self, loader: Iterable | None = None) -> dict[str, Any] | None:
        from nvalchemi_toolkit_b200.training.validation import ValidationLoop

        cfg = self.validation_config
        loader = loader if loader is not None else (cfg.data if cfg is not None else None)
        if loader is None:
            return None
        with ValidationLoop.from_training_strategy(self, cfg) as loop:
            summary = loop.run(loader)
        self.last_validation = summary
        step_schedulers(self._lr_schedulers, self._opt_cfgs, "validation", summary)
        self._run_hooks(TrainingStage.AFTER_VALIDATION, None)
        return summary

    # ---- specs and checkpoints ----------------------------------------------------------------------------------
    def _meta(self) -> dict[str, Any]:
        return {"step_count": self.step_count, "global_step_count": self.global_step_count,
                "batch_count": self.batch_count, "epoch_count": self.epoch_count,
                "epoch_step_count": self.epoch_step_count, "spec": self.to_spec_dict()}

    def _apply_meta(self, meta: dict[str, Any]) -> None:
        for k in ("step_count", "global_step_count", "batch_count", "epoch_count", "epoch_step_count"):
            setattr(self, k, int(meta.get(k, 0)))

    def to_spec_dict(self) -> dict[str, Any]:
        fn = self.training_fn
        return {"num_epochs": self.num_epochs, "num_steps": self.num_steps,
                "optimizer_configs": {k: [c.to_spec() for c in v] for k, v in self.optimizer_configs.items()},
                "loss_fn": self.loss_fn.to_spec() if self.loss_fn is not None else None,
                "training_fn": type_to_path(fn) if "<locals>" not in getattr(fn, "__qualname__", "<locals>") else None,
                "devices": [str(d) for d in self.devices]}

    @classmethod
    def from_spec_dict(cls, spec: dict[str, Any], models: Any, **overrides: Any) -> "TrainingStrategy":
        kw = dict(num_epochs=spec.get("num_epochs"), num_steps=spec.get("num_steps"),
                  optimizer_configs={k: [OptimizerConfig(**c) for c in v] for k, v in spec["optimizer_configs"].items()},
                  loss_fn=ComposedLossFunction.from_spec(spec["loss_fn"]) if spec.get("loss_fn") else None,
                  training_fn=spec.get("training_fn"), devices=spec.get("devices"))
        kw.update(overrides)
        return cls(models, **kw)

    def save_checkpoint(self, directory: str | Path, asynchronous: bool = False) -> "Path | ckpt.PendingCheckpoint":
        """Rank 0 writes the checkpoint; ``asynchronous=True`` snapshots to host memory and returns a handle whose
        ``wait()`` joins the background writer."""
        if get_rank(self.distributed_manager) != 0:
            return Path(directory)
        return ckpt.save_checkpoint(directory, self.step_count, self.models, self._optimizers, self._lr_schedulers,
                                    self.hooks, self._meta(), optimizer_keys=getattr(self, "_opt_keys", None),
                                    asynchronous=asynchronous)

    def load_checkpoint(self, directory: str | Path, step: int | None = None) -> None:
        """Restore models, optimisers, schedulers, hook states and counters (optimisers are built on demand)."""
        if not self._setup_done:
            self._pending_restore = (directory, step)
            self._apply_meta(ckpt.read_strategy_metadata(directory, step))
            return
        meta = ckpt.load_checkpoint(directory, self.models, self._optimizers, self._lr_schedulers, self.hooks, step=step,
                                    map_location=self.devices[0], optimizer_keys=getattr(self, "_opt_keys", None))
        self._apply_meta(meta)

    restore_checkpoint = load_checkpoint
