# SPDX-License-Identifier: Apache-2.0
"""Import alias for code written against the reference package name.

``install_alias()`` makes ``import nvalchemi`` (and ``from nvalchemi.dynamics import NVE`` ...) resolve to this package,
provided no other distribution named ``nvalchemi`` is importable (it refuses to shadow a real installation unless
``force=True``).  Sub-packages that exist under the same name here (``data``, ``models``, ``dynamics``, ``hooks``,
``training``, ``distributed``) are aliased lazily through a meta-path finder.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

_PREFIX, _TARGET = "nvalchemi", "nvalchemi_toolkit_b200"


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):  # noqa: ANN001
        if fullname == _PREFIX or fullname.startswith(_PREFIX + "."):
            real = _TARGET + fullname[len(_PREFIX):]
            try:
                if importlib.util.find_spec(real) is None:
                    return None
            except ModuleNotFoundError:
                return None
            return importlib.util.spec_from_loader(fullname, self)
        return None

    def create_module(self, spec):  # noqa: ANN001
        module = importlib.import_module(_TARGET + spec.name[len(_PREFIX):])
        sys.modules[spec.name] = module
        return module

    def exec_module(self, module):  # noqa: ANN001
        return None


_finder: _AliasFinder | None = None


def install_alias(force: bool = False) -> None:
    global _finder
    if _finder is not None:
        return
    if not force and _PREFIX not in sys.modules:
        try:
            if importlib.util.find_spec(_PREFIX) is not None:
                raise RuntimeError("a package named 'nvalchemi' is already importable; pass force=True to shadow it")
        except (ImportError, ValueError):
            pass
    _finder = _AliasFinder()
    sys.meta_path.insert(0, _finder)


def remove_alias() -> None:
    global _finder
    if _finder is not None:
        sys.meta_path.remove(_finder)
        _finder = None
    for name in [n for n in sys.modules if n == _PREFIX or n.startswith(_PREFIX + ".")]:
        if getattr(sys.modules[name], "__name__", "").startswith(_TARGET):
            del sys.modules[name]
