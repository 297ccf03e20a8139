# SPDX-License-Identifier: Apache-2.0
"""``FineTuningStrategy``: a ``TrainingStrategy`` that starts from a checkpoint and trains a subset of parameters
(reference ``nvalchemi/training/finetune.py:108-490``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from nvalchemi_toolkit_b200.training.hooks.library import TrainableParameterHook
from nvalchemi_toolkit_b200.training.strategy import TrainingStrategy


#: learning rate given to optimiser configs reused from a pretrained checkpoint (fine-tuning wants a smaller step than
#: the original training run; pass ``optimizer_lr=None`` to keep the original)
DEFAULT_FINETUNE_LR = 1e-4


class FineTuningStrategy(TrainingStrategy):
    def __init__(self, models: Any, *, checkpoint: str | Path | None = None, trainable: list[str] | None = None,
                 strict: bool = False, **kwargs: Any) -> None:
        super().__init__(models, **kwargs)
        if checkpoint is not None:
            self._load_weights(Path(checkpoint), strict)
        if trainable:
            self.register_hook(TrainableParameterHook(trainable))

    def _load_weights(self, path: Path, strict: bool) -> None:
        if path.is_dir():
            from nvalchemi_toolkit_b200.training import checkpoint as ckpt

            ckpt.load_checkpoint(path, self.models, strict=strict)
            return
        payload = torch.load(path, map_location="cpu", weights_only=True)
        state = payload.get("state_dict", payload) if isinstance(payload, dict) else payload
        main = self.models["main"]
        target = getattr(main, "model", main)
        try:
            target.load_state_dict(state, strict=strict)
        except RuntimeError:
            main.load_state_dict(state, strict=strict)

    @classmethod
    def from_pretrained_checkpoint(cls, checkpoint_dir: str | Path, *, checkpoint_index: int = -1, map_location: Any = "cpu",
                                   use_original_loss: bool = False, use_original_opt_class: bool = False,
                                   optimizer_lr: float | None = DEFAULT_FINETUNE_LR, trainable: list[str] | None = None,
                                   module_patches: dict[str, Any] | None = None, **strategy_kwargs: Any) -> "FineTuningStrategy":
        """A NEW fine-tuning run initialised from the models of a checkpoint directory (reference
        ``training/finetune.py:251-395``).  Unlike :meth:`load_checkpoint`, which resumes an interrupted run, nothing but the
        weights is inherited: optimiser and scheduler state, hooks, counters and step / epoch limits start fresh.

        The models are rebuilt from the checkpoint's ``spec.json`` files (one model -> passed as a single model, several ->
        a named mapping).  ``use_original_loss`` / ``use_original_opt_class`` fill ``loss_fn`` / ``optimizer_configs`` from the
        strategy metadata stored with the checkpoint when the caller omits them; reused optimiser configs keep their classes
        and schedulers but take ``optimizer_lr`` as learning rate (``None`` keeps the original).  ``module_patches`` (dotted
        sub-module name -> factory) replaces heads before the optimisers are built; ``trainable`` restricts training to
        parameters matching the patterns."""
        from nvalchemi_toolkit_b200.training import checkpoint as ckpt
        from nvalchemi_toolkit_b200.training.hooks.library import ModulePatchHook
        from nvalchemi_toolkit_b200.training.losses import ComposedLossFunction
        from nvalchemi_toolkit_b200.training.optimizers import OptimizerConfig

        models = ckpt.build_models_from_checkpoint(checkpoint_dir, checkpoint_index, map_location)
        needs_loss = use_original_loss and "loss_fn" not in strategy_kwargs
        needs_opt = use_original_opt_class and "optimizer_configs" not in strategy_kwargs
        if needs_loss or needs_opt:
            try:
                meta = ckpt.read_strategy_metadata(checkpoint_dir, None if checkpoint_index == -1 else checkpoint_index)
            except FileNotFoundError:
                meta = {}
            spec = meta.get("spec") or {}
            if needs_loss:
                if not spec.get("loss_fn"):
                    raise ValueError("cannot reuse the original loss: the checkpoint's strategy metadata holds no loss spec")
                strategy_kwargs["loss_fn"] = ComposedLossFunction.from_spec(spec["loss_fn"])
            if needs_opt:
                raw = spec.get("optimizer_configs")
                if not raw:
                    raise ValueError("cannot reuse the original optimisers: the checkpoint's strategy metadata holds none")
                configs = {k: [OptimizerConfig(**c) for c in v] for k, v in raw.items()}
                if optimizer_lr is not None:
                    for group in configs.values():
                        for c in group:
                            c.kwargs = {**c.kwargs, "lr": optimizer_lr}
                strategy_kwargs["optimizer_configs"] = configs
        hooks = list(strategy_kwargs.pop("hooks", None) or [])
        if module_patches:
            hooks.insert(0, ModulePatchHook(module_patches))
        arg = models["main"] if set(models) == {"main"} else models
        return cls(arg, trainable=trainable, hooks=hooks, **strategy_kwargs)
