# SPDX-License-Identifier: Apache-2.0
"""Pickle-free, JSON-serialisable construction records ("specs").

Reference: ``nvalchemi/training/_spec.py:115-560`` (``BaseSpec``, ``create_model_spec``, ``create_model_spec_from_json``,
``register_type_serializer``): a spec names an importable callable and the keyword arguments to call it with, so that a
checkpoint can rebuild models, optimisers and loss terms without unpickling code objects.

Here a spec is ONE pydantic model (``cls_path``, ``timestamp``, ``kwargs``) instead of a dynamically created model class
per target: the keyword arguments are held in their JSON form (tensors, dtypes, devices, classes and nested specs
included, through the package's serialisation helpers and the registry below) and decoded again by :meth:`BaseSpec.build`.
Arguments are checked against the target's signature when the spec is created, so a misspelt hyperparameter fails at
save time, not at restore time."""
from __future__ import annotations

import datetime as _dt
import inspect
from typing import Any, Callable

from pydantic import BaseModel, ConfigDict, Field, field_validator

from nvalchemi_toolkit_b200 import _serialization as ser

_SERIALIZERS: dict[type, tuple[str, Callable[[Any], Any], Callable[[Any], Any]]] = {}


def register_type_serializer(tp: type, to_json: Callable[[Any], Any], from_json: Callable[[Any], Any], name: str | None = None) -> None:
    """Teach specs a type they cannot store by themselves (e.g. a units object): ``to_json(value)`` must return plain
    JSON data, ``from_json(data)`` the value again.  ``name`` (default: the dotted path of the type) tags the stored form."""
    _SERIALIZERS[tp] = (name or ser.type_to_path(tp), to_json, from_json)


def _encode(value: Any) -> Any:
    if isinstance(value, BaseSpec):
        return {"__spec__": value.model_dump(mode="json")}
    for tp, (tag, to_json, _) in _SERIALIZERS.items():
        if isinstance(value, tp):
            return {"__registered__": tag, "value": to_json(value)}
    if isinstance(value, dict):
        return {str(k): _encode(v) for k, v in value.items()}
    if isinstance(value, tuple):
        return {"__tuple__": [_encode(v) for v in value]}
    if isinstance(value, (list, set, frozenset)):
        return [_encode(v) for v in value]
    return ser.to_jsonable(value)


def _decode(value: Any, build_nested: bool) -> Any:
    if isinstance(value, dict):
        if "__spec__" in value:
            spec = BaseSpec.model_validate(value["__spec__"])
            return spec.build() if build_nested else spec
        if "__registered__" in value:
            for tag, _, from_json in _SERIALIZERS.values():
                if tag == value["__registered__"]:
                    return from_json(value["value"])
            raise KeyError(f"no serializer registered for '{value['__registered__']}' (register_type_serializer)")
        if "__tuple__" in value:
            return tuple(_decode(v, build_nested) for v in value["__tuple__"])
        if any(k in value for k in ("__tensor__", "__dtype__", "__device__", "__type__", "__pydantic__")):
            return ser.from_jsonable(value)
        return {k: _decode(v, build_nested) for k, v in value.items()}
    if isinstance(value, list):
        return [_decode(v, build_nested) for v in value]
    return value


class BaseSpec(BaseModel):
    """``cls_path(**kwargs)``, recorded.  ``build()`` imports the callable and calls it; nested specs (also inside lists,
    tuples and dictionaries) are built first.  ``spec.some_kwarg`` reads a decoded keyword argument."""

    model_config = ConfigDict(arbitrary_types_allowed=True)
    cls_path: str
    timestamp: str = Field(default_factory=lambda: _dt.datetime.now(_dt.timezone.utc).isoformat())
    kwargs: dict[str, Any] = Field(default_factory=dict)

    @field_validator("cls_path")
    @classmethod
    def _importable(cls, path: str) -> str:
        try:
            target = ser.import_from_path(path)
        except (ImportError, AttributeError) as exc:
            raise ValueError(f"cls_path {path!r} cannot be imported: {exc}") from exc
        if not callable(target):
            raise ValueError(f"{path} is not callable")
        return path

    @property
    def target(self) -> Any:
        return ser.import_from_path(self.cls_path)

    def init_kwargs(self, build_nested: bool = False) -> dict[str, Any]:
        """The keyword arguments, decoded (nested specs stay specs unless ``build_nested``)."""
        return {k: _decode(v, build_nested) for k, v in self.kwargs.items()}

    def build(self, **overrides: Any) -> Any:
        kw = self.init_kwargs(build_nested=True)
        kw.update(overrides)
        return self.target(**kw)

    def __getattr__(self, name: str) -> Any:  # only reached when normal lookup fails
        kwargs = self.__dict__.get("kwargs") or {}
        if name in kwargs:
            return _decode(kwargs[name], False)
        raise AttributeError(name)


def create_model_spec(target: Any, **kwargs: Any) -> BaseSpec:
    """Spec for ``target(**kwargs)``.  ``target`` must be importable by dotted path and accept every keyword (a
    ``**kwargs`` catch-all counts); positional-only parameters cannot be recorded and are rejected."""
    path = ser.type_to_path(target)
    try:
        sig = inspect.signature(target)
    except (TypeError, ValueError):
        sig = None
    if sig is not None:
        params = sig.parameters
        bad = [n for n, p in params.items() if p.kind is p.POSITIONAL_ONLY]
        if bad:
            raise TypeError(f"{path} has positional-only parameters {bad}: they cannot be stored as keyword arguments")
        if not any(p.kind is p.VAR_KEYWORD for p in params.values()):
            unknown = sorted(set(kwargs) - set(params))
            if unknown:
                raise TypeError(f"{path} does not accept {unknown}; it accepts {sorted(n for n in params if n != 'self')}")
        missing = [n for n, p in params.items() if p.default is p.empty and p.kind in (p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY)
                   and n not in kwargs and n != "self"]
        if missing:
            raise TypeError(f"{path} needs {missing}")
    return BaseSpec(cls_path=path, kwargs={k: _encode(v) for k, v in kwargs.items()})


def create_model_spec_from_json(spec: "dict[str, Any] | str") -> BaseSpec:
    """A spec from ``spec.model_dump(mode='json')`` / ``spec.model_dump_json()`` output."""
    import json

    data = json.loads(spec) if isinstance(spec, str) else spec
    return BaseSpec.model_validate(data)
