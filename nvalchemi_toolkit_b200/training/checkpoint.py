# SPDX-License-Identifier: Apache-2.0
"""Manifest-based training checkpoints without pickle-dependent structure, in the reference's on-disk layout
(``nvalchemi/training/_checkpoint.py:21-51,175-193,495-532,915-933``)::

    <dir>/manifest.json                          schema_version, checkpoint_index, component name lists, associations
    <dir>/models/<name>/spec.json                {"cls_path", "timestamp", constructor kwargs...}
    <dir>/models/<name>/checkpoints/<N>.pt       state_dict only
    <dir>/optimizers/<model>_optimizer[_i]/spec.json, checkpoints/<N>.pt
    <dir>/schedulers/<model>_scheduler[_i]/spec.json, checkpoints/<N>.pt
    <dir>/hooks/checkpoints/<N>.pt               {"<module>.<QualName>:<occurrence>": state} of checkpointable hooks
    <dir>/strategy.json                          latest strategy metadata (recipe + the five restart counters)
    <dir>/strategy/checkpoints/<N>.json          the same per checkpoint index

``N`` is the checkpoint index (auto-incremented from the manifest).  ``associations`` maps a model name to its
``optimizers`` / ``schedulers`` component names, the ``scheduler_optimizers`` edges and the ``optimizer_parameter_names``
each optimizer holds.  Every ``.pt`` file is read with ``weights_only=True``: hook states must consist of tensors and
plain containers.  Wrapped modules (FSDP) are rejected: only plain / DDP modules are supported, as in the reference
(``_checkpoint.py:127-157``).  Directories written by the earlier layout of this package (``latest`` / ``steps`` in the
manifest) are still readable."""
from __future__ import annotations

import copy
import json
import os
import threading
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

import torch

from nvalchemi_toolkit_b200._serialization import to_jsonable, type_to_path

SCHEMA_VERSION = 1
HOOK_DIR = Path("hooks") / "checkpoints"
STRATEGY_FILE = "strategy.json"
STRATEGY_DIR = Path("strategy") / "checkpoints"
_COUNTERS = ("step_count", "global_step_count", "batch_count", "epoch_count", "epoch_step_count")


def _unwrap(module: torch.nn.Module) -> torch.nn.Module:
    name = type(module).__name__
    if "FullyShardedDataParallel" in name or "FSDP" in name:
        raise TypeError("FSDP-wrapped modules cannot be checkpointed; unwrap them first")
    return module.module if isinstance(module, torch.nn.parallel.DistributedDataParallel) else module


def _now() -> str:
    return datetime.now(timezone.utc).isoformat()


def model_spec(module: torch.nn.Module) -> dict[str, Any]:
    """Constructor spec of a model: ``cls_path`` + ``timestamp`` + JSON-able keyword arguments."""
    m = _unwrap(module)
    if hasattr(m, "checkpoint_spec"):
        raw = m.checkpoint_spec()
        kwargs = raw.get("config", raw.get("kwargs", {}))
        return {"cls_path": raw.get("cls_path", raw.get("cls")), "timestamp": _now(), **to_jsonable(kwargs)}
    return {"cls_path": type_to_path(type(m)), "timestamp": _now(), **to_jsonable(getattr(m, "_init_kwargs", {}))}


def _optimizer_spec(obj: Any) -> dict[str, Any]:
    spec: dict[str, Any] = {"cls_path": type_to_path(type(obj)), "timestamp": _now()}
    defaults = getattr(obj, "defaults", None)
    if isinstance(defaults, dict):
        spec.update({k: v for k, v in to_jsonable(defaults).items()
                     if isinstance(v, (int, float, bool, str, list, type(None)))})
    return spec


def component_names(model_keys: list[str], kind: str) -> list[str]:
    """``<model>_<kind>`` (``<model>_<kind>_<i>`` when a model has several), in the order of ``model_keys``."""
    total: dict[str, int] = {}
    for k in model_keys:
        total[k] = total.get(k, 0) + 1
    seen: dict[str, int] = {}
    out = []
    for k in model_keys:
        i = seen.get(k, 0)
        seen[k] = i + 1
        out.append(f"{k}_{kind}" if total[k] == 1 else f"{k}_{kind}_{i}")
    return out


def hook_state_key(hook: object, occurrence: int) -> str:
    return f"{type(hook).__module__}.{type(hook).__qualname__}:{occurrence}"


def _checkpointable(hooks: Any):
    for h in hooks or []:
        children = getattr(h, "_hooks", None)
        if isinstance(children, (list, tuple)):
            yield from _checkpointable(children)
        if callable(getattr(h, "state_dict", None)) and callable(getattr(h, "load_state_dict", None)):
            yield h


def _keyed_hooks(hooks: Any):
    occ: dict[str, int] = {}
    for h in _checkpointable(hooks):
        cls = f"{type(h).__module__}.{type(h).__qualname__}"
        i = occ.get(cls, 0)
        occ[cls] = i + 1
        yield hook_state_key(h, i), h


def _plain(value: Any) -> Any:
    """Hook state reduced to what ``weights_only=True`` can read back: tensors, numbers, strings, dicts, lists."""
    if isinstance(value, torch.Tensor):
        return value.detach().cpu().clone()
    if isinstance(value, dict):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if value is None or isinstance(value, (bool, int, float, str)):
        return value
    raise TypeError(f"hook state holds a {type(value).__name__}; only tensors and plain containers can be checkpointed")


class CheckpointManifest:
    """``manifest.json``: reads the reference schema (and this package's earlier one), writes the reference schema."""

    def __init__(self, root: str | Path) -> None:
        self.root = Path(root)
        self.path = self.root / "manifest.json"
        self.data: dict[str, Any] = {"schema_version": SCHEMA_VERSION, "checkpoint_index": -1, "models": [],
                                     "optimizers": [], "schedulers": [], "associations": {}}
        self.legacy = False
        if self.path.exists():
            raw = json.loads(self.path.read_text())
            if raw.get("schema_version", 0) > SCHEMA_VERSION:
                raise ValueError(f"checkpoint schema version {raw['schema_version']} is newer than supported ({SCHEMA_VERSION})")
            if "checkpoint_index" not in raw and "latest" in raw:  # earlier layout of this package
                self.legacy = True
                raw["checkpoint_index"] = -1 if raw["latest"] is None else raw["latest"]
            for key in ("models", "checkpoint_index"):
                if key not in raw:
                    raise ValueError(f"manifest.json lacks the required field '{key}'")
            self.data.update(raw)
            self.data["schema_version"] = SCHEMA_VERSION

    @property
    def checkpoint_index(self) -> int:
        return int(self.data["checkpoint_index"])

    def indices(self) -> list[int]:
        """Checkpoint indices present on disk for the first model component."""
        if self.legacy:
            return sorted(int(s) for s in self.data.get("steps", []))
        names = self.data["models"]
        if not names:
            return []
        d = self.root / "models" / names[0] / "checkpoints"
        return sorted(int(f.stem) for f in d.glob("*.pt")) if d.is_dir() else []

    def write(self) -> None:
        self.root.mkdir(parents=True, exist_ok=True)
        out = {k: self.data[k] for k in ("schema_version", "checkpoint_index", "models", "optimizers", "schedulers",
                                         "associations")}
        for k in ("models", "optimizers", "schedulers"):
            out[k] = sorted(out[k])
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps(out, indent=2))
        os.replace(tmp, self.path)  # atomic: a crash never leaves a half-written manifest


def infer_associations(models: dict[str, torch.nn.Module], optimizers: dict[str, Any], schedulers: dict[str, Any]
                       ) -> dict[str, dict[str, Any]]:
    """Model-centric linkage from object identity: an optimizer belongs to every model that owns one of its
    parameters, a scheduler to the models of the optimizer it drives (reference ``_checkpoint.py:728-795``)."""
    assoc: dict[str, dict[str, Any]] = {}
    opt_models: dict[str, list[str]] = {}
    for oname, opt in optimizers.items():
        ids = {id(p) for g in opt.param_groups for p in g["params"]}
        for mname, m in models.items():
            named = [(n, p) for n, p in _unwrap(m).named_parameters() if id(p) in ids]
            if not named:
                continue
            a = assoc.setdefault(mname, {"optimizers": [], "schedulers": []})
            a["optimizers"].append(oname)
            a.setdefault("optimizer_parameter_names", {})[oname] = [f"{mname}.{n}" for n, _ in named]
            opt_models.setdefault(oname, []).append(mname)
    for sname, sched in schedulers.items():
        target = getattr(sched, "optimizer", None)
        for oname, opt in optimizers.items():
            if opt is target:
                for mname in opt_models.get(oname, []):
                    a = assoc.setdefault(mname, {"optimizers": [], "schedulers": []})
                    a["schedulers"].append(sname)
                    a.setdefault("scheduler_optimizers", {})[sname] = oname
    return assoc


def validate_checkpoint(root: str | Path, checkpoint_index: int | None = None) -> list[str]:
    """Problems found in a checkpoint directory (empty list: consistent): missing specs or state files, associations
    that name unknown components."""
    root = Path(root)
    man = CheckpointManifest(root)
    idx = man.checkpoint_index if checkpoint_index is None else checkpoint_index
    problems = []
    for kind in ("models", "optimizers", "schedulers"):
        for name in man.data[kind]:
            d = root / kind / name
            if not man.legacy and not (d / "spec.json").exists():
                problems.append(f"{kind}/{name}: spec.json missing")
            if not (d / "checkpoints" / f"{idx}.pt").exists():
                problems.append(f"{kind}/{name}: checkpoints/{idx}.pt missing")
    for mname, a in man.data.get("associations", {}).items():
        if mname not in man.data["models"]:
            problems.append(f"associations name an unknown model '{mname}'")
        for kind in ("optimizers", "schedulers"):
            for comp in a.get(kind, []):
                if comp not in man.data[kind]:
                    problems.append(f"associations of '{mname}' name an unknown {kind[:-1]} '{comp}'")
    return problems


def host_snapshot(obj: Any) -> Any:
    """Deep copy of a state-dict-like object with every tensor moved to host memory.  CUDA tensors go to pinned buffers
    with non-blocking copies on the current stream; the caller records an event after the call and the writer waits on
    it, so training continues while the copies drain and the files are written from the copies, never from live
    parameters."""
    if isinstance(obj, torch.Tensor):
        if obj.is_cuda:
            out = torch.empty(obj.shape, dtype=obj.dtype, device="cpu", pin_memory=True)
            out.copy_(obj.detach(), non_blocking=True)
            return out
        return obj.detach().clone()
    if isinstance(obj, dict):
        return type(obj)((k, host_snapshot(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return type(obj)(host_snapshot(v) for v in obj)
    return copy.deepcopy(obj)


class PendingCheckpoint:
    """Handle of a checkpoint whose files are being written by a background thread; :meth:`wait` joins it and re-raises
    a failure of the writer."""

    def __init__(self, root: Path, thread: threading.Thread, box: dict[str, Any]) -> None:
        self.root, self._thread, self._box = root, thread, box

    def done(self) -> bool:
        return not self._thread.is_alive()

    def wait(self) -> Path:
        self._thread.join()
        if "error" in self._box:
            raise self._box["error"]
        return self.root


def save_checkpoint(root: str | Path, step: int, models: dict[str, torch.nn.Module], optimizers: list, schedulers: list,
                    hooks: list, strategy_meta: dict[str, Any], optimizer_keys: list[str] | None = None,
                    checkpoint_index: int = -1, asynchronous: bool = False) -> "Path | PendingCheckpoint":
    """Write one checkpoint.  ``optimizers`` / ``schedulers`` are the strategy's flat lists; ``optimizer_keys`` names
    the model each optimizer belongs to (default: the first model).  ``checkpoint_index = -1`` auto-increments.

    ``asynchronous=True`` snapshots every state to (pinned) host memory on the calling thread, returns a
    :class:`PendingCheckpoint` at once and writes the files from a background thread (the reference's checkpoint hook has
    the same switch, ``nvalchemi/training/hooks/checkpoint.py``); the manifest is written last, so a reader never sees an
    index whose files are incomplete."""
    root = Path(root)
    if CheckpointManifest(root).legacy:
        raise ValueError(f"{root} holds a checkpoint in this package's earlier layout; save into a fresh directory")
    grab = host_snapshot if asynchronous else (lambda x: x)
    keys = list(optimizer_keys) if optimizer_keys is not None else [next(iter(models))] * len(optimizers)
    opts = dict(zip(component_names(keys, "optimizer"), optimizers))
    scheds = {n: sc for n, sc in zip(component_names(keys, "scheduler"), schedulers) if sc is not None}
    # ---- collect: everything that touches live objects happens here, on the caller's thread ----------------------
    parts: list[tuple[str, str, Any, dict]] = []
    specs = {}
    for name, m in models.items():
        specs[name] = model_spec(m)
        parts.append(("models", name, grab(_unwrap(m).state_dict()), specs[name]))
    for name, o in opts.items():
        parts.append(("optimizers", name, grab(o.state_dict()), _optimizer_spec(o)))
    for name, sc in scheds.items():
        parts.append(("schedulers", name, grab(sc.state_dict()), {"cls_path": type_to_path(type(sc)), "timestamp": _now()}))
    hook_states = {key: grab(_plain(dict(h.state_dict()))) for key, h in _keyed_hooks(hooks)}
    meta = dict(to_jsonable(strategy_meta))
    meta.setdefault("model_specs", specs)
    associations = infer_associations(dict(models), opts, scheds)

    # ---- commit: files only ---------------------------------------------------------------------------------------
    def commit() -> Path:
        man = CheckpointManifest(root)
        index = man.checkpoint_index + 1 if checkpoint_index == -1 else int(checkpoint_index)
        for kind, name, state, spec in parts:
            d = root / kind / name
            (d / "checkpoints").mkdir(parents=True, exist_ok=True)
            spec_path = d / "spec.json"
            if spec_path.exists():
                old = json.loads(spec_path.read_text())
                if {k: v for k, v in old.items() if k != "timestamp"} != {k: v for k, v in spec.items() if k != "timestamp"}:
                    raise ValueError(f"{kind}/{name}/spec.json disagrees with the component being saved")
            else:
                spec_path.write_text(json.dumps(spec, indent=2))
            torch.save(state, d / "checkpoints" / f"{index}.pt")
            if name not in man.data[kind]:
                man.data[kind].append(name)
        if hook_states:
            (root / HOOK_DIR).mkdir(parents=True, exist_ok=True)
            torch.save(hook_states, root / HOOK_DIR / f"{index}.pt")
        payload = json.dumps(meta, indent=2)
        (root / STRATEGY_FILE).write_text(payload)
        (root / STRATEGY_DIR).mkdir(parents=True, exist_ok=True)
        (root / STRATEGY_DIR / f"{index}.json").write_text(payload)
        man.data["checkpoint_index"] = index
        man.data["associations"] = associations
        man.write()
        return root

    if not asynchronous:
        return commit()
    event = None
    if torch.cuda.is_available():
        event = torch.cuda.Event()
        event.record()
    box: dict[str, Any] = {}

    def work() -> None:
        try:
            if event is not None:
                event.synchronize()  # the device-to-host copies of the snapshot have landed
            commit()
        except BaseException as exc:  # re-raised by PendingCheckpoint.wait()
            box["error"] = exc

    th = threading.Thread(target=work, name="checkpoint-writer", daemon=True)
    th.start()
    return PendingCheckpoint(root, th, box)



def build_models_from_checkpoint(root: str | Path, checkpoint_index: int | None = None, map_location: Any = "cpu",
                                 strict: bool = True) -> dict[str, torch.nn.Module]:
    """Instantiate every model of a checkpoint from its ``spec.json`` (``cls_path`` + constructor keywords) and load the
    weights of the chosen index (default: the manifest's latest).  The classes must be importable; nothing but tensors is
    unpickled."""
    from nvalchemi_toolkit_b200._serialization import import_from_path

    root = Path(root)
    man = CheckpointManifest(root)
    idx = man.checkpoint_index if checkpoint_index in (None, -1) else int(checkpoint_index)
    models: dict[str, torch.nn.Module] = {}
    for name in man.data["models"]:
        spec = json.loads((root / "models" / name / "spec.json").read_text())
        kwargs = {k: v for k, v in spec.items() if k not in ("cls_path", "timestamp")}
        module = import_from_path(spec["cls_path"])(**kwargs)
        state_file = root / "models" / name / "checkpoints" / f"{idx}.pt"
        if not state_file.exists():
            raise FileNotFoundError(f"model '{name}' has no weights for checkpoint index {idx} under {root}")
        _unwrap(module).load_state_dict(torch.load(state_file, map_location=map_location, weights_only=True), strict=strict)
        models[name] = module
    if not models:
        raise FileNotFoundError(f"{root} holds no model component")
    return models


def read_strategy_metadata(root: str | Path, checkpoint_index: int | None = None) -> dict[str, Any]:
    root = Path(root)
    man = CheckpointManifest(root)
    idx = man.checkpoint_index if checkpoint_index is None else checkpoint_index
    if man.legacy:
        return json.loads((root / "strategy" / f"{idx}.json").read_text())
    f = root / STRATEGY_DIR / f"{idx}.json"
    if not f.exists():
        f = root / STRATEGY_FILE
    return json.loads(f.read_text()) if f.exists() else {}


#: ``(component, saved_spec, current_spec) -> None``; raise to veto a restore
CheckpointValidator = Callable[[str, Mapping[str, Any], Mapping[str, Any]], None]


def same_class_validator(component: str, saved: Mapping[str, Any], current: Mapping[str, Any]) -> None:
    """Veto restoring weights into a different class than the one that was saved."""
    if saved and saved.get("cls_path") != current.get("cls_path"):
        raise ValueError(f"{component}: checkpoint holds {saved.get('cls_path')}, the model being restored is "
                         f"{current.get('cls_path')}")


def load_checkpoint(root: str | Path, models: dict[str, torch.nn.Module], optimizers: list | None = None,
                    schedulers: list | None = None, hooks: list | None = None, step: int | None = None,
                    map_location: Any = "cpu", strict: bool = True, optimizer_keys: list[str] | None = None,
                    validators: "Sequence[CheckpointValidator] | None" = None) -> dict[str, Any]:
    """Restores states in place and returns the strategy metadata (counters) of the chosen checkpoint index
    (``step``; default: the manifest's latest).

    ``validators``: callables ``(component, saved_spec, current_spec) -> None`` run for every model BEFORE any state is
    touched (``component`` is ``"models/<name>"``; the specs are the ``spec.json`` record and :func:`model_spec` of the
    model being restored); one that raises aborts the load with nothing modified (reference ``_checkpoint.py:101``).
    :func:`same_class_validator` is a ready-made one."""
    root = Path(root)
    man = CheckpointManifest(root)
    idx = man.checkpoint_index if step is None else int(step)
    if idx < 0 or (man.indices() and idx not in man.indices()):
        raise FileNotFoundError(f"no checkpoint with index {idx} under {root}")

    def read(f: Path) -> Any:
        return torch.load(f, map_location=map_location, weights_only=True)

    if validators:
        for name, m in models.items():
            spec_file = root / "models" / name / "spec.json"
            saved = json.loads(spec_file.read_text()) if spec_file.exists() else {}
            current = model_spec(_unwrap(m))
            for check in validators:
                check(f"models/{name}", saved, current)
    for name, m in models.items():
        f = root / "models" / name / "checkpoints" / f"{idx}.pt"
        if f.exists():
            _unwrap(m).load_state_dict(read(f), strict=strict)
    optimizers, schedulers = list(optimizers or []), list(schedulers or [])
    if man.legacy:
        opt_names = [str(i) for i in range(len(optimizers))]
        sched_names = [str(i) for i in range(len(schedulers))]
    else:
        keys = list(optimizer_keys) if optimizer_keys is not None else [next(iter(models))] * len(optimizers)
        opt_names = component_names(keys, "optimizer")
        sched_names = component_names(keys, "scheduler")  # the scheduler list is aligned with the optimizer list
    for name, o in zip(opt_names, optimizers):
        f = root / "optimizers" / name / "checkpoints" / f"{idx}.pt"
        if f.exists():
            o.load_state_dict(read(f))
    for name, s in zip(sched_names, schedulers):
        f = root / "schedulers" / name / "checkpoints" / f"{idx}.pt"
        if s is not None and f.exists():
            s.load_state_dict(read(f))
    if man.legacy:
        for h in hooks or []:
            if hasattr(h, "load_state_dict"):
                f = root / "hooks" / getattr(h, "checkpoint_name", type(h).__name__) / f"{idx}.pt"
                if f.exists():
                    h.load_state_dict(read(f))
    else:
        f = root / HOOK_DIR / f"{idx}.pt"
        if f.exists():
            saved = read(f)
            for key, h in _keyed_hooks(hooks):
                if key in saved:
                    h.load_state_dict(saved[key])
    return read_strategy_metadata(root, idx)
