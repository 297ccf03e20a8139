# SPDX-License-Identifier: Apache-2.0
"""Bounds-checked debug mode for the native operators.

The kernels trust their index arguments (batch indices, CSR pointers, sender lists, halo routing tables): a bad index is
an out-of-range access on the device, which surfaces late or not at all.  With this mode on
(``NVALCHEMI_B200_DEBUG_BOUNDS=1`` in the environment, or :func:`enable`), every call that goes through the package's
operator proxy first validates those arguments on the host, against the sizes of the tensors they index, and raises an
``IndexError`` that names the operator, the argument and the offending value BEFORE the kernel is launched.  The checks
read the index tensors back (one reduction each), so the mode is for debugging and CI on small cases, not for timed runs.
It plays the role of the reference's Warp ``verify_*`` / debug-mode bounds checking (``wp.config.mode = "debug"`` in its
test configuration) for kernels that are hand-written here.

Rules are keyed on argument NAMES of the operator schemas, so a new operator that follows the naming conventions
(``batch_idx``, ``eptr``, ``esend``, ``home_rank`` ...) is covered without registering anything.
"""
from __future__ import annotations

import os
from typing import Any, Callable

import torch

_enabled = bool(int(os.environ.get("NVALCHEMI_B200_DEBUG_BOUNDS", "0") or 0))
num_checked = 0  # operator calls validated so far (tests read it)


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def _fail(op: str, arg: str, what: str) -> None:
    raise IndexError(f"nvalchemi::{op}: argument '{arg}' {what}")


def _range(op: str, arg: str, t: torch.Tensor | None, lo: int, hi: int | None, mask: torch.Tensor | None = None) -> None:
    """Every (selected) entry of ``t`` lies in ``[lo, hi)``."""
    if t is None or t.numel() == 0:
        return
    v = t if mask is None else t[mask]
    if v.numel() == 0:
        return
    mn, mx = int(v.min()), int(v.max())
    if mn < lo:
        _fail(op, arg, f"holds {mn}, below the lower bound {lo}")
    if hi is not None and mx >= hi:
        _fail(op, arg, f"holds {mx}, outside [{lo}, {hi})")


def _monotone(op: str, arg: str, t: torch.Tensor | None, limit: int | None = None) -> None:
    if t is None or t.numel() == 0:
        return
    if int(t[0]) < 0:
        _fail(op, arg, f"starts at {int(t[0])} (negative offset)")
    if t.numel() > 1 and bool((t[1:] < t[:-1]).any()):
        _fail(op, arg, "is not non-decreasing")
    if limit is not None and int(t[-1]) > limit:
        _fail(op, arg, f"ends at {int(t[-1])}, past the {limit} rows it indexes")


def _rows(x: Any) -> int | None:
    return int(x.shape[0]) if isinstance(x, torch.Tensor) and x.dim() >= 1 else None


_PER_SYSTEM = ("dt", "alpha", "kT", "temperature", "friction", "cells", "cell", "kinetic_tensors", "shift", "scale", "A", "Q")


def _num_systems(b: dict[str, Any]) -> int | None:
    if isinstance(b.get("num_systems"), int):
        return int(b["num_systems"])
    for k in _PER_SYSTEM:
        t = b.get(k)
        if isinstance(t, torch.Tensor) and t.dim() >= 1:
            if k in ("cell", "cells") and t.dim() == 2:
                return 1
            return int(t.shape[0])
    return None


def check(op: str, schema: Any, args: tuple, kwargs: dict) -> None:
    """Validate the index arguments of one operator call (no-op for operators without any)."""
    global num_checked
    names = [a.name for a in schema.arguments]
    b: dict[str, Any] = dict(zip(names, args))
    b.update(kwargs)
    num_checked += 1
    n_atoms = next((r for r in (_rows(b.get(k)) for k in ("positions", "pos", "velocities", "x")) if r is not None), None)

    bi = b.get("batch_idx")
    if isinstance(bi, torch.Tensor):
        if n_atoms is not None and bi.numel() < n_atoms:
            _fail(op, "batch_idx", f"has {bi.numel()} entries for {n_atoms} rows")
        _range(op, "batch_idx", bi if n_atoms is None else bi[:n_atoms], 0, _num_systems(b))

    for ptr_name in ("source_batch_ptr", "dest_batch_ptr", "batch_ptr"):
        _monotone(op, ptr_name, b.get(ptr_name) if isinstance(b.get(ptr_name), torch.Tensor) else None)

    esend, eptr = b.get("esend"), b.get("eptr")
    if isinstance(eptr, torch.Tensor) and isinstance(esend, torch.Tensor) and op != "csr_fill":
        _monotone(op, "eptr", eptr, int(esend.numel()))
    if isinstance(esend, torch.Tensor) and op not in ("csr_fill", "mark_used_senders"):
        n_send_rows = n_atoms
        if isinstance(eptr, torch.Tensor) and eptr.numel():
            esend = esend[: int(eptr[-1])]
        _range(op, "esend", esend, 0, n_send_rows)
    if op == "mark_used_senders":
        _range(op, "esend", b["esend"][: int(b["n_edges"])], 0, int(b["n_owned"]) + int(b["used"].numel()))

    nm = b.get("neighbor_matrix")
    if isinstance(nm, torch.Tensor) and n_atoms is not None:
        _range(op, "neighbor_matrix", nm, 0, n_atoms + 1)  # the fill value n marks an empty slot
        nn = b.get("num_neighbors")
        if isinstance(nn, torch.Tensor):
            _range(op, "num_neighbors", nn, 0, int(nm.shape[1]) + 1)

    world = None
    for k in ("src_ptrs", "dst_ptrs", "ptrs", "u_ptrs", "ghost_src_ptrs"):
        if isinstance(b.get(k), torch.Tensor):
            world = int(b[k].numel())
            break
    for k in ("home_rank", "peer", "ghost_home_rank"):
        if isinstance(b.get(k), torch.Tensor):
            _range(op, k, b[k], 0, world)
    for k in ("home_row", "peer_row", "dst_row", "ghost_home_row"):
        if isinstance(b.get(k), torch.Tensor):
            hi = _rows(b.get("buf")) if (k == "dst_row" and op == "halo_pull_add_rows") else None
            _range(op, k, b[k], 0, hi)
    if op in ("halo_pull_rows", "halo_push_add_rows"):
        t = b.get("dst") if op == "halo_pull_rows" else b.get("src")
        need = int(b["row0"]) + int(b["home_rank"].numel())
        if _rows(t) is not None and need > _rows(t):
            _fail(op, "row0", f"+ {int(b['home_rank'].numel())} ghost rows = {need} exceeds the {_rows(t)} rows of the buffer")

    if op == "copy_rows":
        _range(op, "src_rows", b["src_rows"], 0, _rows(b["src"]))
        _range(op, "dst_rows", b["dst_rows"], 0, _rows(b["dst"]))
    if op == "segmented_reduce":
        _range(op, "idx", b["idx"], 0, int(b["num_segments"]))
    if op == "segmented_copy_planned":
        plan, sp = b["plan"], b["source_batch_ptr"]
        lens = (sp[1:] - sp[:-1])[: plan.numel()]
        go = plan >= 0
        if bool(go.any()) and int((plan + lens)[go].max()) > _rows(b["dest"]):
            _fail(op, "plan", f"places a segment past the {_rows(b['dest'])} rows of the destination")
    sp = b.get("species")
    if isinstance(sp, torch.Tensor):
        _range(op, "species", sp, 0, None)


def wrap(name: str, fn: Callable) -> Callable:
    """Operator callable that validates first while the mode is on (used by the operator proxy)."""
    schema = fn.default._schema

    def checked(*a: Any, **k: Any) -> Any:
        if _enabled:
            check(name, schema, a, k)
        return fn(*a, **k)

    checked.__name__ = name
    return checked
