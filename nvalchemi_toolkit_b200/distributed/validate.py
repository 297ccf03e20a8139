# SPDX-License-Identifier: Apache-2.0
"""Checks that a model evaluates identically with and without domain decomposition.

Reference: ``nvalchemi/distributed/validate/*.py`` (``trace_and_validate``: reference run → spawn N ranks → diff →
suggested fixes; halo-completeness check).  Here: :func:`check_halo_completeness` verifies that every owned atom sees
the same number of neighbours in its padded sub-domain as in the full system; :func:`trace_and_validate` runs the
model once on the whole batch and once on ``world_size`` gloo ranks on CPU, compares energy / forces / stress, and, if
they differ, tries the usual repairs (a deeper halo; the other consolidation mode) and reports which one works.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, replace
from types import SimpleNamespace
from typing import Any, Callable

import torch
import torch.distributed as dist


@dataclass
class ValidationReport:
    ok: bool
    max_abs_diff: dict[str, float]
    world_size: int
    spec_name: str
    suggestion: str | None = None
    attempts: list[dict[str, Any]] = field(default_factory=list)
    #: the spec that reproduces the single-process result (declared, inferred or repaired); ``None`` when none did
    spec: Any = None
    #: what the trace of the single-process run saw, when the spec was inferred
    trace: str | None = None
    #: one sentence: what to do with this report
    next_action: str = ""

    def spec_dict(self) -> dict | None:
        """The working spec as plain data (``MLIPSpec.from_dict`` restores it; ``MLIPSpec.save`` writes it to a file)."""
        return None if self.spec is None else self.spec.to_dict()

    def __str__(self) -> str:
        head = "PASS" if self.ok else "FAIL"
        diffs = ", ".join(f"{k} {v:.3e}" for k, v in self.max_abs_diff.items())
        tail = f"; suggestion: {self.suggestion}" if self.suggestion else ""
        tail += f"\n  next: {self.next_action}" if self.next_action else ""
        return f"[{head}] {self.spec_name} on {self.world_size} ranks: {diffs}{tail}"


def check_halo_completeness(sharded: Any, cutoff: float, global_batch: Any) -> tuple[bool, int]:
    """``(complete, number of owned atoms with missing neighbours)`` for one rank's padded sub-domain."""
    from nvalchemi_toolkit_b200 import neighbors as nb

    padded = sharded.padded_batch()
    nb.compute_neighbors(padded, cutoff)
    full = global_batch.clone()
    nb.compute_neighbors(full, cutoff)
    want = full.num_neighbors[sharded.global_ids.to(full.device)]
    got = padded.num_neighbors[: sharded.n_owned]
    missing = int((got.cpu() != want.cpu()).sum())
    return missing == 0, missing


def _reference(model: Any, batch: Any) -> dict:
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    return {k: v.detach().clone() for k, v in model(batch).items() if isinstance(v, torch.Tensor)}


def _worker(rank: int, world: int, port: int, q: Any, model_factory: Callable, batch_factory: Callable, cfg_kwargs: dict,
            spec: Any) -> None:
    from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, ShardedBatch, ShardTensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        model, batch = model_factory(), batch_factory()
        cfg = DomainConfig(**cfg_kwargs)
        use = spec if spec is not None else model.distribution_spec()
        sh = ShardedBatch.from_batch(batch, cfg, use)
        out = DistributedModel(model, cfg, use)(sh)
        res = {}
        for k, v in out.items():
            if not isinstance(v, torch.Tensor):
                continue
            res[k] = (ShardTensor(v, sh).full_tensor() if v.dim() >= 1 and v.shape[0] == sh.n_owned and k not in
                      use.extensive_outputs else v).tolist()
        complete, missing = check_halo_completeness(sh, cfg.cutoff, batch) if model.model_config.neighbor_config else (True, 0)
        if rank == 0:
            q.put((res, missing))
        else:
            q.put((None, missing))
    finally:
        dist.destroy_process_group()


def _spawn(world: int, port: int, model_factory: Callable, batch_factory: Callable, cfg_kwargs: dict, spec: Any
           ) -> tuple[dict, int]:
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, model_factory, batch_factory, cfg_kwargs, spec))
             for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    res = next(r for r, _ in got if r is not None)
    return res, sum(m for _, m in got)


def _diff(ref: dict, res: dict, keys: tuple[str, ...]) -> dict[str, float]:
    out = {}
    for k in keys:
        if k in ref and k in res:
            a, b = ref[k].double().reshape(-1), torch.tensor(res[k], dtype=torch.float64).reshape(-1)
            out[k] = float((a - b).abs().max()) if a.numel() == b.numel() else float("inf")
    return out


def trace_and_validate(model_factory: Callable, batch_factory: Callable, world_size: int = 2, *, cutoff: float,
                       skin: float = 0.0, spec: Any = None, atol: float = 1e-6, port: int = 29733,
                       keys: tuple[str, ...] = ("energy", "forces", "stress"), auto_fix: bool = True,
                       infer: bool | None = None) -> ValidationReport:
    """``model_factory`` / ``batch_factory`` must be importable top-level callables (they run in spawned processes).

    The spec under test is ``spec``, else the one the model declares (``distribution_spec()``), else one inferred from
    a trace of the single-process run (:func:`~nvalchemi_toolkit_b200.distributed.infer_spec.infer_spec`).  ``infer=True``
    always traces and uses the declared spec only as a prior (its non-default fields win)."""
    from nvalchemi_toolkit_b200.distributed.infer_spec import infer_spec
    from nvalchemi_toolkit_b200.distributed.spec import Consolidation

    model = model_factory()
    ref = _reference(model, batch_factory())
    declared = spec
    if declared is None and hasattr(model, "distribution_spec"):
        try:
            declared = model.distribution_spec()
        except NotImplementedError:
            declared = None
    trace_text = None
    if infer or (infer is None and declared is None):
        base, summary = infer_spec(model, batch_factory(), prior=declared)
        trace_text = summary.describe()
    elif declared is None:
        raise ValueError("the model declares no distribution spec: pass spec=... or allow inference (infer=None / True)")
    else:
        base = declared
    cfg = {"cutoff": cutoff, "skin": skin}
    attempts = []

    def attempt(s: Any, label: str, p: int) -> tuple[bool, dict[str, float]]:
        res, missing = _spawn(world_size, p, model_factory, batch_factory, cfg, s)
        d = _diff(ref, res, keys)
        ok = all(v <= atol for v in d.values())
        attempts.append({"label": label, "ok": ok, "diff": d, "atoms_with_missing_neighbors": missing})
        return ok, d

    ok, d = attempt(base, "inferred spec" if trace_text is not None else "declared spec", port)
    suggestion = None
    working = base if ok else None
    if not ok and auto_fix:
        fixes = [(replace(base, message_passes=base.message_passes + 1), f"message_passes={base.message_passes + 1} (deeper halo)")]
        other = Consolidation.WEIGHTED_ENERGY if base.consolidation == Consolidation.DIRECT_MASKED else Consolidation.DIRECT_MASKED
        fixes.append((replace(base, consolidation=other), f"consolidation={other.value}"))
        if not base.refresh_per_layer:
            fixes.append((replace(base, refresh_per_layer=True),
                          "refresh_per_layer=True (ghost rows refreshed before every gather, sums over owned rows only)"))
        for i, (s, label) in enumerate(fixes):
            try:
                fixed, _ = attempt(s, label, port + 1 + i)
            except Exception as exc:  # noqa: BLE001 - a repair that cannot run is just not a repair
                attempts.append({"label": label, "ok": False, "error": repr(exc)})
                continue
            if fixed:
                suggestion, working = label, s
                break
    if ok:
        action = ("use the inferred spec: return it from the wrapper's distribution_spec() or save it with "
                  "report.spec.save(path)") if trace_text is not None else "nothing to do: the declared spec reproduces the single-process result"
    elif working is not None:
        action = f"change the spec: {suggestion}; the repaired spec is report.spec"
    else:
        missing = max((a.get("atoms_with_missing_neighbors", 0) or 0) for a in attempts)
        action = (f"{missing} owned atoms miss neighbours in their sub-domain: increase the ghost depth (cutoff / skin / "
                  "message_passes)" if missing else
                  "no automatic repair matched: run layer_diff(...) to find the first layer whose owned rows deviate")
    return ValidationReport(ok, d, world_size, base.name, suggestion, attempts, working, trace_text, action)


# ---- layer-by-layer comparison (reference ``nvalchemi/distributed/validate/layer_diagnostics.py``) ---------------
def _capture_node_outputs(model: Any, n_rows: int) -> tuple[dict[str, torch.Tensor], list]:
    """Forward hooks that keep, per named sub-module, its first tensor output with ``n_rows`` rows."""
    store: dict[str, torch.Tensor] = {}
    handles = []

    def make(name: str) -> Callable:
        def hook(_m: Any, _inp: Any, out: Any) -> None:
            t = out if isinstance(out, torch.Tensor) else next((o for o in out if isinstance(o, torch.Tensor)), None) \
                if isinstance(out, (tuple, list)) else None
            if isinstance(t, torch.Tensor) and t.dim() >= 1 and t.shape[0] == n_rows and name not in store:
                store[name] = t.detach().clone()
        return hook

    for name, mod in model.named_modules():
        if name:
            handles.append(mod.register_forward_hook(make(name)))
    return store, handles


def _layer_worker(rank: int, world: int, port: int, q: Any, model_factory: Callable, batch_factory: Callable,
                  cfg_kwargs: dict, spec: Any) -> None:
    from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, ShardedBatch, ShardTensor

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        model, batch = model_factory(), batch_factory()
        cfg = DomainConfig(**cfg_kwargs)
        use = spec if spec is not None else model.distribution_spec()
        sh = ShardedBatch.from_batch(batch, cfg, use)
        store, handles = _capture_node_outputs(model, sh.n_owned + sh.n_ghost)
        DistributedModel(model, cfg, use)(sh)
        for h in handles:
            h.remove()
        names = sorted(store)  # the same modules fire on every rank: the gathers below stay aligned
        full = {k: ShardTensor(store[k][: sh.n_owned].contiguous(), sh).full_tensor().tolist() for k in names}
        q.put((full if rank == 0 else None, 0))
    finally:
        dist.destroy_process_group()


def layer_diff(model_factory: Callable, batch_factory: Callable, world_size: int = 2, *, cutoff: float, skin: float = 0.0,
               spec: Any = None, atol: float = 1e-6, port: int = 29761) -> list[dict]:
    """Per sub-module, the largest difference between its per-atom output in a single-process evaluation and in the
    decomposed one (owned rows, gathered in global order), in execution order of the single-process run.  The first
    entry with ``ok = False`` is where the decomposition starts to deviate (a layer that needs refreshed ghost rows, a
    reduction that counts ghosts, ...).  Factories must be importable top-level callables."""
    import torch.multiprocessing as mp

    model, batch = model_factory(), batch_factory()
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    store, handles = _capture_node_outputs(model, batch.num_nodes)
    model(batch)
    for h in handles:
        h.remove()
    order = list(store)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_worker, args=(r, world_size, port, q, model_factory, batch_factory,
                                                     {"cutoff": cutoff, "skin": skin}, spec)) for r in range(world_size)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world_size)]
    for p in procs:
        p.join(timeout=30)
    res = next(r for r, _ in got if r is not None)
    report = []
    for name in order:
        if name not in res:
            report.append({"module": name, "ok": False, "max_abs_diff": float("inf"), "note": "not captured under decomposition"})
            continue
        a, b = store[name].double(), torch.tensor(res[name], dtype=torch.float64)
        d = float((a - b).abs().max()) if a.shape == b.shape else float("inf")
        report.append({"module": name, "ok": d <= atol, "max_abs_diff": d})
    return report


# ---- scripted helpers (reference ``nvalchemi/distributed/validate/scripted_diagnostics.py``) -----------------------
@dataclass
class ScriptedOpReport:
    """TorchScript objects reachable from a model.  The dispatch mode of the distributed forward is a
    ``TorchFunctionMode``: it does not see the tensor operations INSIDE a scripted module or function, so a scripted
    message-passing block needs an adapter (``JitAdapter`` for a module-level function, ``ModuleForwardAdapter`` for a
    scripted sub-module) before ``refresh_per_layer`` can be trusted."""

    modules: list[str] = field(default_factory=list)     # dotted names of scripted sub-modules
    functions: list[str] = field(default_factory=list)   # "package.module.name" of scripted module-level functions

    @property
    def found(self) -> bool:
        return bool(self.modules or self.functions)

    def advice(self) -> str:
        if not self.found:
            return "no scripted code found: gathers and scatters are visible to the dispatch mode"
        lines = []
        if self.functions:
            lines.append("scripted functions (declare JitAdapter(module, name, mode='marshal', node_inputs=..., node_outputs=...) "
                         "or give a plain-Python replacement): " + ", ".join(self.functions))
        if self.modules:
            lines.append("scripted sub-modules (declare ModuleForwardAdapter(cls, node_inputs=..., node_outputs=...)): "
                         + ", ".join(self.modules))
        return "; ".join(lines)


def detect_scripted_ops(model: Any) -> ScriptedOpReport:
    """Scan ``model`` for scripted sub-modules and the Python modules that define its sub-module classes for scripted
    module-level functions."""
    import sys

    report = ScriptedOpReport()
    if not isinstance(model, torch.nn.Module):
        return report
    seen_py: set[str] = set()
    for name, sub in model.named_modules():
        if isinstance(sub, torch.jit.ScriptModule):
            report.modules.append(name or type(sub).__name__)
        mod_name = type(sub).__module__
        if mod_name in seen_py or mod_name.startswith("torch."):
            continue
        seen_py.add(mod_name)
        py = sys.modules.get(mod_name)
        for attr, value in (vars(py).items() if py is not None else ()):
            if isinstance(value, torch.jit.ScriptFunction):
                report.functions.append(f"{mod_name}.{attr}")
    report.functions.sort()
    return report


#: names under which the reference exports the report types
TraceReport = ValidationReport
Attempt = dict
