# SPDX-License-Identifier: Apache-2.0
"""``FineTuningStrategy``: a ``TrainingStrategy`` that starts from a checkpoint and trains a subset of parameters
(reference ``nvalchemi/training/finetune.py:108-490``)."""
from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from nvalchemi_toolkit_b200.training.hooks.library import TrainableParameterHook
from nvalchemi_toolkit_b200.training.strategy import TrainingStrategy


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
