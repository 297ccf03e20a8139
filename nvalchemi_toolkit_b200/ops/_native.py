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
    _register_fakes()
    return LIB_PATH


_fakes_done = False


def _register_fakes() -> None:
    """``torch.library.register_fake`` for the operators dynamics code calls, so that a function using them can be traced
    (``torch.compile(fullgraph=True)``, ``make_fx``) without entering the kernels: they become opaque graph nodes, as the
    reference's custom ops are (``nvalchemi/dynamics/_ops/velocity_verlet.py:50-143``).  Runs once, after the library
    has been loaded."""
    global _fakes_done
    if _fakes_done:
        return
    _fakes_done = True
    nothing = [
        "vv_position_update", "vv_velocity_finalize", "langevin_half_step", "langevin_finalize", "nhc_chain_update",
        "nhc_velocity_half_step", "nhc_position_update", "compute_kinetic_tensor", "affine_rows_", "_fire_step_op",
        "velocity_shift_scale", "fire2_step", "segmented_copy_planned", "compute_put_fit_mask_per_system", "put_masked_per_system", "defrag_per_system",
        "compute_put_fit_mask_segmented", "put_masked_segmented", "defrag_segmented"]
    shaped = {
        "compute_kinetic_energy": lambda v, m, b, n: v.new_empty(n),
        "nhc_chain_scalar": lambda ke2, *a, **k: torch.empty_like(ke2),
        "momentum_sums": lambda v, m, b, n: v.new_empty(n, 4),
        "wrap_positions": lambda p, *a, **k: torch.empty_like(p),
    }
    for name in nothing:
        shaped[name] = lambda *a, **k: None
    for name, fn in shaped.items():
        try:
            torch.library.register_fake(f"nvalchemi::{name}")(fn)
        except (RuntimeError, ValueError):  # operator absent from an older build of the library
            pass


def available() -> bool:
    """True when the native library is loaded (loads it on first call if present)."""
    global _loaded
    if _loaded is None:
        if os.path.exists(LIB_PATH):
            torch.ops.load_library(LIB_PATH)
            _loaded = True
            _register_fakes()
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
