# SPDX-License-Identifier: Apache-2.0
"""Pickle-free (de)serialisation helpers for dtypes, devices, tensors and types.

Equivalent in scope to the reference's ``nvalchemi/_serialization.py:29-326``:
JSON-friendly encodings plus a dotted-path importer restricted to importable
module attributes, used by config specs and checkpoints so that nothing on disk
requires ``pickle`` to interpret.
"""
from __future__ import annotations

import importlib
from typing import Any

import torch

_DTYPES = {
    str(d).replace("torch.", ""): d
    for d in (
        torch.float16, torch.bfloat16, torch.float32, torch.float64,
        torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool,
        torch.complex64, torch.complex128,
    )
}


def dtype_to_str(dtype: torch.dtype) -> str:
    return str(dtype).replace("torch.", "")


def str_to_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = name.replace("torch.", "")
    if key not in _DTYPES:
        raise ValueError(f"Unknown torch dtype name: {name!r}")
    return _DTYPES[key]


def device_to_str(device: torch.device | str) -> str:
    return str(torch.device(device))


def str_to_device(name: str | torch.device) -> torch.device:
    return torch.device(name)


def tensor_to_json(t: torch.Tensor | None) -> dict[str, Any] | None:
    """Encode a tensor as ``{"dtype", "shape", "data"}`` (nested lists)."""
    if t is None:
        return None
    cpu = t.detach().cpu()
    return {"dtype": dtype_to_str(cpu.dtype), "shape": list(cpu.shape), "data": cpu.tolist()}


def tensor_from_json(obj: Any) -> torch.Tensor | None:
    if obj is None or isinstance(obj, torch.Tensor):
        return obj
    if isinstance(obj, dict) and "data" in obj:
        t = torch.tensor(obj["data"], dtype=str_to_dtype(obj.get("dtype", "float32")))
        return t.reshape(obj["shape"]) if "shape" in obj else t
    return torch.as_tensor(obj)


def type_to_path(obj: Any) -> str:
    """Dotted import path (``module.qualname``) of a class or function."""
    mod = getattr(obj, "__module__", None)
    qual = getattr(obj, "__qualname__", None)
    if mod is None or qual is None or "<locals>" in qual:
        raise ValueError(f"{obj!r} has no importable dotted path")
    return f"{mod}.{qual}"


def import_from_path(path: str) -> Any:
    """Resolve ``pkg.mod.Attr`` (or ``pkg.mod:Attr``) by import + getattr only."""
    path = path.replace(":", ".")
    parts = path.split(".")
    for cut in range(len(parts) - 1, 0, -1):
        try:
            obj: Any = importlib.import_module(".".join(parts[:cut]))
        except ImportError:
            continue
        for attr in parts[cut:]:
            obj = getattr(obj, attr)
        return obj
    raise ImportError(f"Cannot import {path!r}")


def to_jsonable(value: Any) -> Any:
    """Recursively convert a config value into JSON-compatible structures."""
    if isinstance(value, torch.Tensor):
        return {"__tensor__": tensor_to_json(value)}
    if isinstance(value, torch.dtype):
        return {"__dtype__": dtype_to_str(value)}
    if isinstance(value, torch.device):
        return {"__device__": str(value)}
    if isinstance(value, type) or callable(value) and hasattr(value, "__qualname__"):
        return {"__type__": type_to_path(value)}
    if isinstance(value, dict):
        return {str(k): to_jsonable(v) for k, v in value.items()}
    if isinstance(value, (list, tuple, set, frozenset)):
        return [to_jsonable(v) for v in value]
    if hasattr(value, "model_dump"):
        return {"__pydantic__": type_to_path(type(value)), "fields": to_jsonable(value.model_dump())}
    return value


def from_jsonable(value: Any) -> Any:
    if isinstance(value, dict):
        if "__tensor__" in value:
            return tensor_from_json(value["__tensor__"])
        if "__dtype__" in value:
            return str_to_dtype(value["__dtype__"])
        if "__device__" in value:
            return torch.device(value["__device__"])
        if "__type__" in value:
            return import_from_path(value["__type__"])
        if "__pydantic__" in value:
            return import_from_path(value["__pydantic__"])(**from_jsonable(value["fields"]))
        return {k: from_jsonable(v) for k, v in value.items()}
    if isinstance(value, list):
        return [from_jsonable(v) for v in value]
    return value


class SerializableClass:
    """Mixin: ``to_spec()`` / ``from_spec()`` round-trip through constructor kwargs.

    A subclass records its constructor arguments in ``self._init_kwargs`` (or
    overrides ``_spec_kwargs``); the spec is a JSON-safe dict with the class path.
    """

    def _spec_kwargs(self) -> dict[str, Any]:
        return dict(getattr(self, "_init_kwargs", {}))

    def to_spec(self) -> dict[str, Any]:
        return {"cls": type_to_path(type(self)), "kwargs": to_jsonable(self._spec_kwargs())}

    @staticmethod
    def from_spec(spec: dict[str, Any]) -> Any:
        cls = import_from_path(spec["cls"])
        return cls(**from_jsonable(spec.get("kwargs", {})))
