# SPDX-License-Identifier: Apache-2.0
"""Former home of the profiling hooks (reference ``nvalchemi/dynamics/hooks/profiling.py:1-33`` keeps the same alias).
They live in :mod:`nvalchemi_toolkit_b200.hooks` now; importing them from here still works and warns once."""
import warnings


def __getattr__(name: str):
    if name in ("TorchProfilerHook", "StageTimingHook"):
        warnings.warn(f"import {name} from nvalchemi_toolkit_b200.hooks", DeprecationWarning, stacklevel=2)
        import nvalchemi_toolkit_b200.hooks as hooks

        return getattr(hooks, name)
    if name == "ProfilerHook":
        raise AttributeError("ProfilerHook was removed; use TorchProfilerHook or StageTimingHook")
    raise AttributeError(name)
