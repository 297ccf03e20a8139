# SPDX-License-Identifier: Apache-2.0
"""Optional third-party dependencies and a decorator that demands them.

Same role as the reference's ``nvalchemi/_optional.py:27-162``: each enum member
knows its import name and install hint; ``.require`` wraps a callable (or class)
so that calling it without the dependency raises a readable ``ImportError``
instead of an ``AttributeError`` deep inside an adapter.
"""
from __future__ import annotations

import functools
import importlib
import importlib.util
from enum import Enum
from typing import Any, Callable, TypeVar

F = TypeVar("F", bound=Callable[..., Any])


class MissingDependencyError(ImportError):
    """Raised when an optional dependency is needed but not importable."""


class OptionalDependency(Enum):
    ASE = ("ase", "pip install ase")
    PYMATGEN = ("pymatgen", "pip install pymatgen")
    MACE = ("mace", "pip install mace-torch")
    AIMNET = ("aimnet", "pip install aimnet")
    TENSORBOARD = ("tensorboard", "pip install tensorboard")
    UMA = ("fairchem.core", "pip install fairchem-core")
    CUEQUIVARIANCE = ("cuequivariance", "pip install cuequivariance")
    CUEQUIVARIANCE_OPS = ("cuequivariance_ops_torch", "pip install cuequivariance-ops-torch-cu12")
    ZSTD = ("zstandard", "pip install zstandard")
    YAML = ("yaml", "pip install pyyaml")

    @property
    def import_name(self) -> str:
        return self.value[0]

    @property
    def install_hint(self) -> str:
        return self.value[1]

    def is_available(self) -> bool:
        try:
            return importlib.util.find_spec(self.import_name) is not None
        except (ImportError, ValueError):
            return False

    def import_module(self) -> Any:
        if not self.is_available():
            raise MissingDependencyError(self._message())
        return importlib.import_module(self.import_name)

    def _message(self, what: str | None = None) -> str:
        subject = f"{what} needs" if what else "This feature needs"
        return (
            f"{subject} the optional dependency '{self.import_name}', which is not "
            f"installed. Install it with: {self.install_hint}"
        )

    def require(self, obj: F) -> F:
        """Decorate a function or class so use without the dependency fails clearly."""
        dep = self
        if isinstance(obj, type):
            orig_init = obj.__init__

            @functools.wraps(orig_init)
            def _init(self_: Any, *a: Any, **k: Any) -> None:
                if not dep.is_available():
                    raise MissingDependencyError(dep._message(obj.__name__))
                orig_init(self_, *a, **k)

            obj.__init__ = _init  # type: ignore[misc]
            return obj  # type: ignore[return-value]

        @functools.wraps(obj)
        def _wrapped(*a: Any, **k: Any) -> Any:
            if not dep.is_available():
                raise MissingDependencyError(dep._message(getattr(obj, "__qualname__", str(obj))))
            return obj(*a, **k)

        return _wrapped  # type: ignore[return-value]
