# SPDX-License-Identifier: Apache-2.0
"""Locating, building and loading the sm_100a extension (``_C``).

All CUDA/C++ sources live in ``nvalchemi_toolkit_b200/csrc``.  They are compiled
into ONE shared library placed inside the package directory
(``nvalchemi_toolkit_b200/_C.so``), registered through ``TORCH_LIBRARY`` and loaded
with ``torch.ops.load_library``; kernels are then reachable as
``torch.ops.nvalchemi.*``.  On a machine that has a CUDA device the library is
mandatory: a missing library raises instead of silently running a PyTorch
fallback.  On CPU-only machines the pure-torch implementations in
``nvalchemi_toolkit_b200.ops`` are used when the library is absent.
"""
from __future__ import annotations

import glob
import os
import shutil
import sys

import torch

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "_C.so")
_loaded: bool | None = None

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source for sm_100a into ``_C.so`` (cross-compiles without a GPU)."""
    if not force and not _stale():
        return LIB_PATH
    from torch.utils import cpp_extension

    build_dir = os.path.join(PKG_DIR, "_build")
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    cpp_extension.load(
        name="nvalchemi_b200_C",
        sources=sources(),
        extra_cflags=["-O3", "-fopenmp", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-lineinfo", "-std=c++17", "--extended-lambda", "-Xcompiler", "-fopenmp", "-Xptxas", "-v"] + ARCH_FLAGS,
        extra_ldflags=["-L/usr/lib/x86_64-linux-gnu", "-l:libgomp.so.1"],
        extra_include_paths=[CSRC],
        build_directory=build_dir,
        is_python_module=False,
        verbose=verbose,
    )
    built = os.path.join(build_dir, "nvalchemi_b200_C.so")
    shutil.copyfile(built, LIB_PATH)
    global _loaded
    _loaded = True  # cpp_extension.load already registered the ops in this process
    return LIB_PATH


def available() -> bool:
    """True when the native library is loaded (loads it on first call if present)."""
    global _loaded
    if _loaded is None:
        if os.path.exists(LIB_PATH):
            torch.ops.load_library(LIB_PATH)
            _loaded = True
        else:
            _loaded = False
            if torch.cuda.is_available() and not os.environ.get("NVALCHEMI_B200_ALLOW_FALLBACK"):
                raise RuntimeError(
                    f"CUDA device present but the native extension {LIB_PATH} is missing. "
                    "Build it with `python -m nvalchemi_toolkit_b200.ops.build`."
                )
    return bool(_loaded)


def require(t: torch.Tensor | None = None) -> bool:
    """Should the native kernel be used for tensor ``t``?  Raises on CUDA tensors without the library."""
    ok = available()
    if t is not None and t.is_cuda and not ok:
        raise RuntimeError("native extension not loaded but a CUDA tensor was passed")
    return ok


if __name__ == "__main__":  # python -m nvalchemi_toolkit_b200.ops._native
    print(build(force="--force" in sys.argv, verbose=True))
