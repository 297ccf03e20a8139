# SPDX-License-Identifier: Apache-2.0
"""Manifest-based training checkpoints without pickle-dependent structure.

Directory layout (same as the reference, ``nvalchemi/training/_checkpoint.py:21-51``)::

    <dir>/manifest.json
    <dir>/models/<name>/spec.json              constructor spec (class path + JSON kwargs)
    <dir>/models/<name>/checkpoints/<step>.pt  state_dict only
    <dir>/optimizers/<i>/spec.json, checkpoints/<step>.pt
    <dir>/schedulers/<i>/...
    <dir>/hooks/<name>/<step>.pt               states of CheckpointableHook hooks
    <dir>/strategy/<step>.json                 counters and the strategy spec

``manifest.json`` lists components, the available steps and ``latest``.  Wrapped modules (FSDP) are rejected: only
plain / DDP modules are supported, as in the reference (``_checkpoint.py:127-157``)."""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any

import torch

from nvalchemi_toolkit_b200._serialization import to_jsonable, type_to_path

SCHEMA_VERSION = 1


def _unwrap(module: torch.nn.Module) -> torch.nn.Module:
    name = type(module).__name__
    if "FullyShardedDataParallel" in name or "FSDP" in name:
        raise TypeError("FSDP-wrapped modules cannot be checkpointed; unwrap them first")
    return module.module if isinstance(module, torch.nn.parallel.DistributedDataParallel) else module


def model_spec(module: torch.nn.Module) -> dict[str, Any]:
    m = _unwrap(module)
    if hasattr(m, "checkpoint_spec"):
        return m.checkpoint_spec()
    return {"cls": type_to_path(type(m)), "kwargs": to_jsonable(getattr(m, "_init_kwargs", {}))}


class CheckpointManifest:
    def __init__(self, root: str | Path) -> None:
        self.root = Path(root)
        self.path = self.root / "manifest.json"
        self.data: dict[str, Any] = {"schema_version": SCHEMA_VERSION, "models": [], "optimizers": [], "schedulers": [],
                                     "hooks": [], "steps": [], "latest": None}
        if self.path.exists():
            self.data = json.loads(self.path.read_text())
            if self.data.get("schema_version", 0) > SCHEMA_VERSION:
                raise ValueError("checkpoint written by a newer schema version")

    def write(self) -> None:
        self.root.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps(self.data, indent=1))
        os.replace(tmp, self.path)  # atomic: a crash never leaves a half-written manifest


def save_checkpoint(root: str | Path, step: int, models: dict[str, torch.nn.Module], optimizers: list, schedulers: list,
                    hooks: list, strategy_meta: dict[str, Any]) -> Path:
    root = Path(root)
    man = CheckpointManifest(root)

    def put(kind: str, name: str, state: Any, spec: dict | None) -> None:
        d = root / kind / name
        (d / "checkpoints").mkdir(parents=True, exist_ok=True)
        if spec is not None:
            (d / "spec.json").write_text(json.dumps(spec, indent=1))
        torch.save(state, d / "checkpoints" / f"{step}.pt")
        if name not in man.data[kind]:
            man.data[kind].append(name)

    for name, m in models.items():
        put("models", name, _unwrap(m).state_dict(), model_spec(m))
    for i, o in enumerate(optimizers):
        put("optimizers", str(i), o.state_dict(), {"cls": type_to_path(type(o))})
    for i, s in enumerate(schedulers):
        if s is not None:
            put("schedulers", str(i), s.state_dict(), {"cls": type_to_path(type(s))})
    for h in hooks:
        if hasattr(h, "state_dict") and hasattr(h, "load_state_dict"):
            name = getattr(h, "checkpoint_name", type(h).__name__)
            d = root / "hooks" / name
            d.mkdir(parents=True, exist_ok=True)
            torch.save(dict(h.state_dict()), d / f"{step}.pt")
            if name not in man.data["hooks"]:
                man.data["hooks"].append(name)
    (root / "strategy").mkdir(parents=True, exist_ok=True)
    (root / "strategy" / f"{step}.json").write_text(json.dumps(to_jsonable(strategy_meta), indent=1))
    if step not in man.data["steps"]:
        man.data["steps"].append(step)
    man.data["latest"] = step
    man.write()
    return root


def load_checkpoint(root: str | Path, models: dict[str, torch.nn.Module], optimizers: list | None = None,
                    schedulers: list | None = None, hooks: list | None = None, step: int | None = None,
                    map_location: Any = "cpu", strict: bool = True) -> dict[str, Any]:
    """Restores states in place and returns the strategy metadata (counters) of the chosen step."""
    root = Path(root)
    man = CheckpointManifest(root)
    step = man.data["latest"] if step is None else step
    if step is None or step not in man.data["steps"]:
        raise FileNotFoundError(f"no checkpoint for step {step} under {root}")
    for name, m in models.items():
        f = root / "models" / name / "checkpoints" / f"{step}.pt"
        if f.exists():
            _unwrap(m).load_state_dict(torch.load(f, map_location=map_location, weights_only=True), strict=strict)
    for i, o in enumerate(optimizers or []):
        f = root / "optimizers" / str(i) / "checkpoints" / f"{step}.pt"
        if f.exists():
            o.load_state_dict(torch.load(f, map_location=map_location, weights_only=True))
    for i, s in enumerate(schedulers or []):
        f = root / "schedulers" / str(i) / "checkpoints" / f"{step}.pt"
        if s is not None and f.exists():
            s.load_state_dict(torch.load(f, map_location=map_location, weights_only=True))
    for h in hooks or []:
        if hasattr(h, "load_state_dict"):
            f = root / "hooks" / getattr(h, "checkpoint_name", type(h).__name__) / f"{step}.pt"
            if f.exists():
                h.load_state_dict(torch.load(f, map_location=map_location, weights_only=False))
    return json.loads((root / "strategy" / f"{step}.json").read_text())
