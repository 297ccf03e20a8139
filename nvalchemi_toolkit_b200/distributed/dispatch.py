# SPDX-License-Identifier: Apache-2.0
"""Per-layer ghost refresh for UNMODIFIED message-passing models.

Reference: ``nvalchemi/distributed/_core/shard_tensor.py:677-934`` (dim-0 ``index_select`` / ``__getitem__`` /
``scatter_add_`` / ``index_add_`` on node tensors are classified into ghost refresh, halo correction and owned-only
per-system reduction) and ``_core/adapter.py`` (``OpAdapter``, ``FunctionAdapter``, ``MethodAdapter``,
``ModuleForwardAdapter``, ``AdapterRegistry``: the same treatment at the boundary of opaque custom ops).

The reference attaches this behaviour to a tensor subclass.  Here it is a ``TorchFunctionMode`` that is active only
inside the distributed forward: node tensors stay plain tensors and the mode keeps a weak table of the ones whose
ghost rows are out of date ("stale").  With a ghost layer ONE cutoff deep (instead of one per message pass):

* a scatter along dim 0 that produces a node tensor (``n_owned + n_ghost`` rows) leaves owned rows complete and ghost
  rows partial: the result is marked stale (and, if the policy folds, ghost partial sums first go to their owners);
* staleness propagates through every op that maps a stale node tensor to another node tensor;
* a gather along dim 0 from a stale node tensor first refreshes the ghost rows from their owners
  (:func:`~nvalchemi_toolkit_b200.distributed.ops.halo_forward`, whose backward returns ghost-row gradients);
* a scatter along dim 0 FROM a node tensor into something smaller (per-system sums) only counts owned rows.
"""
from __future__ import annotations

import contextvars
import functools
import weakref
from typing import Any, Callable, Iterable

import torch
from torch.overrides import TorchFunctionMode

from nvalchemi_toolkit_b200.distributed.storage_policy import RefreshOnlyHaloPolicy

__all__ = ["HaloDispatchMode", "current_dispatch", "OpAdapter", "FunctionAdapter", "MethodAdapter",
           "ModuleForwardAdapter", "AdapterRegistry", "PythonAdapter", "JitAdapter", "AdapterStatus"]

_ACTIVE: contextvars.ContextVar["HaloDispatchMode | None"] = contextvars.ContextVar("nva_halo_dispatch", default=None)

_GATHERS = {"index_select", "__getitem__", "gather", "take_along_dim"}
_SCATTERS = {"index_add_", "index_add", "scatter_add_", "scatter_add", "scatter_reduce_", "scatter_reduce", "index_put_",
             "index_put", "index_reduce_", "index_reduce"}


def current_dispatch() -> "HaloDispatchMode | None":
    return _ACTIVE.get()


class _WeakIds:
    """Set of live tensors keyed by identity."""

    def __init__(self) -> None:
        self._d: dict[int, Any] = {}

    def add(self, t: torch.Tensor) -> None:
        key = id(t)
        self._d[key] = weakref.ref(t, lambda _r, k=key, d=self._d: d.pop(k, None))

    def discard(self, t: torch.Tensor) -> None:
        self._d.pop(id(t), None)

    def __contains__(self, t: object) -> bool:
        r = self._d.get(id(t))
        return r is not None and r() is t


def _tensors(obj: Any) -> Iterable[torch.Tensor]:
    if isinstance(obj, torch.Tensor):
        yield obj
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            yield from _tensors(o)
    elif isinstance(obj, dict):
        for o in obj.values():
            yield from _tensors(o)


class HaloDispatchMode(TorchFunctionMode):
    def __init__(self, halo: Any, n_owned: int, policy: Any = None, group: Any = None, global_ids: Any = None) -> None:
        super().__init__()
        self.halo, self.n_owned, self.group, self.global_ids = halo, int(n_owned), group, global_ids
        self.n_padded = int(n_owned) + int(halo.n_ghost)
        self.policy = policy if policy is not None else RefreshOnlyHaloPolicy()
        self._stale = _WeakIds()
        self._fresh: dict[int, tuple[Any, int, torch.Tensor]] = {}
        self.stats = {"refreshes": 0, "folds": 0, "masked_reductions": 0}
        self._token: Any = None

    # ---- bookkeeping ------------------------------------------------------------------------------------------
    def is_node(self, t: Any) -> bool:
        return isinstance(t, torch.Tensor) and t.dim() >= 1 and t.shape[0] == self.n_padded and self.halo.n_ghost > 0

    def is_stale(self, t: Any) -> bool:
        return isinstance(t, torch.Tensor) and t in self._stale

    def mark_stale(self, t: torch.Tensor) -> None:
        if self.is_node(t):
            self._stale.add(t)

    def refresh(self, x: torch.Tensor) -> torch.Tensor:
        """Node tensor with current ghost rows (cached per source tensor and version)."""
        hit = self._fresh.get(id(x))
        if hit is not None and hit[0]() is x and hit[1] == x._version:
            return hit[2]
        fresh = self.policy.replicate(x, self)
        self.stats["refreshes"] += 1
        key = id(x)
        self._fresh[key] = (weakref.ref(x, lambda _r, k=key, d=self._fresh: d.pop(k, None)), x._version, fresh)
        return fresh

    def owned_mask(self, like: torch.Tensor) -> torch.Tensor:
        m = torch.zeros(self.n_padded, dtype=like.dtype, device=like.device)
        m[: self.n_owned] = 1
        return m.reshape((self.n_padded,) + (1,) * (like.dim() - 1))

    def __enter__(self) -> "HaloDispatchMode":
        self._token = _ACTIVE.set(self)
        return super().__enter__()

    def __exit__(self, *exc: Any) -> Any:
        _ACTIVE.reset(self._token)
        return super().__exit__(*exc)

    # ---- interception -------------------------------------------------------------------------------------------
    def __torch_function__(self, func: Callable, types: Any, args: tuple = (), kwargs: dict | None = None) -> Any:
        kwargs = kwargs or {}
        name = getattr(func, "__name__", "")
        if name in _GATHERS and args and self.is_stale(args[0]) and self._gathers_rows(name, args, kwargs):
            args = (self.refresh(args[0]),) + tuple(args[1:])
            return func(*args, **kwargs)  # edge-level result: nothing to track
        if name in _SCATTERS and args:
            return self._scatter(func, name, args, kwargs)
        out = func(*args, **kwargs)
        if any(self.is_stale(t) for t in _tensors(args)) or any(self.is_stale(t) for t in _tensors(kwargs)):
            for t in _tensors(out):
                self.mark_stale(t)
        return out

    @staticmethod
    def _dim_is_zero(t: torch.Tensor, dim: Any) -> bool:
        return isinstance(dim, int) and (dim == 0 or dim == -t.dim())

    def _gathers_rows(self, name: str, args: tuple, kwargs: dict) -> bool:
        x = args[0]
        if name == "__getitem__":
            idx = args[1]
            first = idx[0] if isinstance(idx, tuple) and idx else idx
            return isinstance(first, torch.Tensor) and first.dtype in (torch.int64, torch.int32)
        dim = args[1] if len(args) > 1 else kwargs.get("dim")
        return self._dim_is_zero(x, dim)

    def _scatter(self, func: Callable, name: str, args: tuple, kwargs: dict) -> Any:
        target = args[0]
        if name.startswith("index_put"):
            indices = args[1] if len(args) > 1 else kwargs.get("indices")
            src = args[2] if len(args) > 2 else kwargs.get("values")
            accumulate = args[3] if len(args) > 3 else kwargs.get("accumulate", False)
            rows = bool(accumulate) and isinstance(indices, (tuple, list)) and len(indices) >= 1
            src_pos, src_key = 2, "values"
        else:
            dim = args[1] if len(args) > 1 else kwargs.get("dim")
            rows = isinstance(target, torch.Tensor) and self._dim_is_zero(target, dim)
            src_pos = 3
            src_key = "source" if name.startswith("index_") else "src"
            src = args[3] if len(args) > 3 else kwargs.get(src_key)
        if not rows or not isinstance(target, torch.Tensor):
            out = func(*args, **kwargs)
            if any(self.is_stale(t) for t in _tensors(args)):
                for t in _tensors(out):
                    self.mark_stale(t)
            return out
        if self.is_node(src) and not self.is_node(target):
            # per-system (or any coarser) reduction of a node tensor: ghost rows are copies of atoms counted elsewhere
            masked = src * self.owned_mask(src)
            self.stats["masked_reductions"] += 1
            if len(args) > src_pos:
                args = tuple(args[:src_pos]) + (masked,) + tuple(args[src_pos + 1:])
            else:
                kwargs = dict(kwargs, **{src_key: masked})
            return func(*args, **kwargs)
        out = func(*args, **kwargs)
        if self.is_node(out):
            if getattr(self.policy, "scatter_mode", "local") != "local":
                folded = self.policy.fold(out, self)
                self.stats["folds"] += 1
                if name.endswith("_"):
                    out.copy_(folded)  # in-place scatter: callers keep using the target object
                else:
                    out = folded
            self.mark_stale(out)
        return out


# ---- adapters: the same treatment at the boundary of opaque operators --------------------------------------------
class OpAdapter:
    """Wraps a callable the dispatch mode cannot see into (a fused gather+scatter kernel, a scripted function).

    ``node_inputs``: positions or keyword names of node tensors the op READS by neighbour index: stale ones are
    refreshed before the call.  ``node_outputs``: positions (in the returned tuple; ``0`` for a single tensor) of node
    tensors the op SCATTERS into: they are folded per the policy and marked stale.  ``reduce_outputs``: outputs that
    are per-system sums over local atoms and must be summed over the ranks.  Outside a distributed forward the wrapped
    callable is called as is."""

    def __init__(self, node_inputs: Iterable[int | str] = (), node_outputs: Iterable[int] = (),
                 reduce_outputs: Iterable[int] = ()) -> None:
        self.node_inputs, self.node_outputs, self.reduce_outputs = tuple(node_inputs), tuple(node_outputs), tuple(reduce_outputs)

    def wrap(self, fn: Callable) -> Callable:
        adapter = self

        @functools.wraps(fn)
        def wrapped(*args: Any, **kwargs: Any) -> Any:
            mode = current_dispatch()
            if mode is None:
                return fn(*args, **kwargs)
            args = list(args)
            for key in adapter.node_inputs:
                if isinstance(key, int) and key < len(args) and mode.is_stale(args[key]):
                    args[key] = mode.refresh(args[key])
                elif isinstance(key, str) and mode.is_stale(kwargs.get(key)):
                    kwargs[key] = mode.refresh(kwargs[key])
            out = fn(*args, **kwargs)
            single = not isinstance(out, (tuple, list))
            outs = [out] if single else list(out)
            for i in adapter.node_outputs:
                if i < len(outs) and mode.is_node(outs[i]):
                    if getattr(mode.policy, "scatter_mode", "local") != "local":
                        outs[i] = mode.policy.fold(outs[i], mode)
                    mode.mark_stale(outs[i])
            for i in adapter.reduce_outputs:
                if i < len(outs) and isinstance(outs[i], torch.Tensor):
                    from nvalchemi_toolkit_b200.distributed.ops import distributed_all_reduce

                    outs[i] = distributed_all_reduce(outs[i], mode.group)
            return outs[0] if single else type(out)(outs)

        wrapped.__wrapped_by_adapter__ = adapter  # type: ignore[attr-defined]
        return wrapped


class FunctionAdapter(OpAdapter):
    """Adapter installed over ``getattr(module, name)`` (a module-level function or a ``torch.ops`` namespace entry)."""

    def __init__(self, owner: Any, name: str, **kw: Any) -> None:
        super().__init__(**kw)
        self.owner, self.name = owner, name

    def install(self) -> Callable:
        original = getattr(self.owner, self.name)
        setattr(self.owner, self.name, self.wrap(original))
        return original

    def restore(self, original: Callable) -> None:
        setattr(self.owner, self.name, original)


class MethodAdapter(FunctionAdapter):
    """Adapter over a method of a class; positions in ``node_inputs`` count ``self`` as argument 0."""


class ModuleForwardAdapter(MethodAdapter):
    """Adapter over ``forward`` of an ``nn.Module`` subclass (e.g. an interaction block backed by a fused kernel)."""

    def __init__(self, module_cls: type, **kw: Any) -> None:
        super().__init__(module_cls, "forward", **kw)


class PythonAdapter:
    """Replace a module-level helper ``module_path.attr_name`` for the duration of a distributed forward (reference
    ``_core/adapter.py:827-900``): helpers of third-party packages whose single-process assumptions break on a padded
    sub-domain (an output size read from ``index[-1] + 1``, a sum over all local rows that must skip ghost rows).
    ``replacement`` receives the same arguments as the original; it may be set after construction (a wrapper's
    ``distributed_setup`` knows the partition) but must be there when the adapter is installed."""

    kind = "python"

    def __init__(self, module_path: str, attr_name: str, replacement: Callable | None = None) -> None:
        self.module_path, self.attr_name, self.replacement = module_path, attr_name, replacement
        self.install_site = _call_site()

    def target(self) -> str:
        return f"{self.module_path}.{self.attr_name}"

    def _owner(self) -> Any:
        import importlib

        return importlib.import_module(self.module_path)

    def _replacement_for(self, original: Callable) -> Callable:
        if self.replacement is None:
            raise RuntimeError(f"{type(self).__name__}({self.target()}): no replacement was given before install")
        return self.replacement

    def install(self) -> Callable:
        owner = self._owner()
        original = getattr(owner, self.attr_name)
        setattr(owner, self.attr_name, self._replacement_for(original))
        return original

    def restore(self, original: Callable) -> None:
        setattr(self._owner(), self.attr_name, original)


class JitAdapter(PythonAdapter):
    """The same for a ``torch.jit.script``-ed helper, which the dispatch mode cannot see into.  ``mode="eager"`` swaps
    in ``replacement`` (a plain-Python restatement whose gathers and scatters the mode does see); ``mode="marshal"``
    keeps the scripted function and treats it as an opaque operator: stale node inputs (``node_inputs``) are refreshed
    before the call, node outputs (``node_outputs``) are folded / marked stale after it, exactly like
    :class:`OpAdapter` (reference ``_core/adapter.py:717-825``)."""

    kind = "jit"

    def __init__(self, module_path: str, attr_name: str, replacement: Callable | None = None, mode: str = "eager",
                 node_inputs: Iterable[int | str] = (), node_outputs: Iterable[int] = (), reduce_outputs: Iterable[int] = ()) -> None:
        if mode not in ("eager", "marshal"):
            raise ValueError(f"mode must be 'eager' or 'marshal', got {mode!r}")
        if mode == "eager" and replacement is None:
            raise ValueError("mode='eager' needs a replacement")
        super().__init__(module_path, attr_name, replacement)
        self.mode = mode
        self._op = OpAdapter(node_inputs, node_outputs, reduce_outputs)

    def _replacement_for(self, original: Callable) -> Callable:
        return self._op.wrap(original) if self.mode == "marshal" else super()._replacement_for(original)


def _call_site() -> str:
    """``file:line`` of the first frame outside this module (where an adapter was declared)."""
    import inspect

    for frame in inspect.stack()[2:]:
        if frame.filename != __file__:
            return f"{frame.filename.rsplit('/', 1)[-1]}:{frame.lineno}"
    return ""


class AdapterStatus:
    """One adapter's life-cycle state, as listed by :meth:`AdapterRegistry.list_active`: ``kind`` (``op`` / ``python`` /
    ``jit``), ``target`` (what was replaced), ``state`` (``pending``, ``installed``, ``restored``, ``failed``), ``error``
    (text of the exception when the install failed) and ``install_site`` (where the adapter was declared)."""

    def __init__(self, kind: str, target: str, state: str = "pending", error: str | None = None, install_site: str = "") -> None:
        self.kind, self.target, self.state, self.error, self.install_site = kind, target, state, error, install_site

    def __repr__(self) -> str:
        tail = f", error={self.error!r}" if self.error else ""
        return f"AdapterStatus({self.kind} {self.target}: {self.state}{tail})"


class AdapterRegistry:
    """Installs a set of adapters for the duration of a ``with`` block (or between ``install`` / ``restore``)."""

    def __init__(self, adapters: Iterable[Any] = ()) -> None:
        self.adapters = list(adapters)
        self._originals: list[tuple[Any, Callable]] = []
        self._status: dict[int, AdapterStatus] = {}
        for a in self.adapters:
            self._track(a)

    def _track(self, a: Any) -> AdapterStatus:
        target = a.target() if hasattr(a, "target") else f"{getattr(getattr(a, 'owner', None), '__name__', a.__class__.__name__)}.{getattr(a, 'name', '?')}"
        st = AdapterStatus(getattr(a, "kind", "op"), target, install_site=getattr(a, "install_site", ""))
        self._status[id(a)] = st
        return st

    def register(self, adapter: Any) -> "AdapterRegistry":
        self.adapters.append(adapter)
        self._track(adapter)
        return self

    def install(self) -> None:
        """Install every adapter; if one fails, those already installed are put back and the error is re-raised (the
        failed one is listed with ``state="failed"``)."""
        if self._originals:
            return
        for a in self.adapters:
            st = self._status[id(a)]
            try:
                self._originals.append((a, a.install()))
                st.state, st.error = "installed", None
            except Exception as exc:  # noqa: BLE001 - recorded, then re-raised after the roll-back
                st.state, st.error = "failed", f"{type(exc).__name__}: {exc}"
                self.restore()
                raise

    def restore(self) -> None:
        for a, original in reversed(self._originals):
            a.restore(original)
            self._status[id(a)].state = "restored"
        self._originals.clear()

    def list_active(self) -> list[AdapterStatus]:
        """Status of every registered adapter (what is swapped in this process right now, and what failed)."""
        return [self._status[id(a)] for a in self.adapters]

    def __enter__(self) -> "AdapterRegistry":
        self.install()
        return self

    def __exit__(self, *exc: Any) -> None:
        self.restore()
