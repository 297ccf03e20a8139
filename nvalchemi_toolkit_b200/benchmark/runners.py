# SPDX-License-Identifier: Apache-2.0
"""Config-driven benchmark runners: model forward and NVT dynamics, single process or domain-decomposed.

Reference: ``benchmark/distributed/_benchmark_common.py:620-2016``, ``benchmark_dd_model_forward.py``,
``benchmark_dd_nvt.py``: build a synthetic system, gate on force equivalence between the decomposed and the
single-process evaluation, time steps with CUDA events (wall clock on CPU), shrink the system and retry after an
out-of-memory error, and emit one JSON record per case.
"""
from __future__ import annotations

import json
import time
from dataclasses import asdict, dataclass, field
from types import SimpleNamespace
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200._serialization import import_from_path


@dataclass
class BenchmarkCase:
    name: str
    system: str = "fcc_cu"
    size: int = 4
    model: str = "nvalchemi_toolkit_b200.models.lj.LennardJonesModelWrapper"
    model_kwargs: dict[str, Any] = field(default_factory=lambda: {"epsilon": 0.0104, "sigma": 3.4, "cutoff": 8.5})
    mode: str = "forward"          # "forward" | "nvt"
    steps: int = 10
    warmup: int = 3
    dt: float = 1.0
    temperature: float = 300.0
    skin: float = 0.5
    dtype: str = "float32"
    device: str = "auto"
    distributed: bool = False       # evaluate through DomainParallel / DistributedModel on the active process group
    check_forces: bool = True
    force_tolerance: float = 1e-4
    min_size: int = 1


class StepTimer:
    """CUDA-event timing of a region on the current stream (``time.perf_counter`` on CPU)."""

    def __init__(self, device: torch.device) -> None:
        self.cuda = device.type == "cuda"
        self.samples: list[float] = []

    def __enter__(self) -> "StepTimer":
        if self.cuda:
            self._a, self._b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            self._a.record()
        else:
            self._t = time.perf_counter()
        return self

    def __exit__(self, *exc: Any) -> None:
        if self.cuda:
            self._b.record()
            torch.cuda.synchronize()
            self.samples.append(self._a.elapsed_time(self._b))
        else:
            self.samples.append((time.perf_counter() - self._t) * 1e3)


def _device(case: BenchmarkCase) -> torch.device:
    if case.device != "auto":
        return torch.device(case.device)
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _max_over_ranks(ms: float, device: torch.device) -> float:
    _, world = _world()
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device if dist.get_backend() == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _build_model(case: BenchmarkCase, device: torch.device, dtype: torch.dtype) -> Any:
    model = import_from_path(case.model)(**case.model_kwargs)
    if isinstance(model, torch.nn.Module):
        model = model.to(device=device)
        if any(True for _ in model.parameters()):
            model = model.to(dtype)
    model.model_config.active_outputs = {"energy", "forces"}
    return model


def force_equivalence(model: Any, batch: Any, case: BenchmarkCase) -> float:
    """Largest force difference between the domain-decomposed and the single-process evaluation (0 without a group)."""
    from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, ShardedBatch, ShardTensor

    ref_batch = batch.clone()
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=ref_batch), None)
    ref = model(ref_batch)["forces"].detach()
    nc = model.model_config.neighbor_config
    cfg = DomainConfig(cutoff=nc.cutoff if nc is not None else 1.0, skin=case.skin)
    sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
    out = DistributedModel(model, cfg)(sh)
    full = ShardTensor(out["forces"], sh).full_tensor()
    return float((full - ref).abs().max())


def run_case(case: BenchmarkCase) -> dict[str, Any]:
    device = _device(case)
    dtype = getattr(torch, case.dtype)
    rank, world = _world()
    size = case.size
    while True:
        oom, result = False, None
        try:
            result = _run(case, size, device, dtype, rank, world)
        except torch.cuda.OutOfMemoryError:
            oom = True
            torch.cuda.empty_cache()
        if world > 1:  # one rank out of memory means every rank skips this size (nobody waits in a collective alone)
            flag = torch.tensor([1.0 if oom else 0.0], device=device if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            oom = bool(flag > 0)
        if not oom:
            return result
        if size <= case.min_size:
            return {"name": case.name, "status": "oom", "size": size}
        size = max(case.min_size, size - max(1, size // 4))  # shrink by a quarter and try again


def _run(case: BenchmarkCase, size: int, device: torch.device, dtype: torch.dtype, rank: int, world: int) -> dict[str, Any]:
    from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel, DistributedModel, ShardedBatch
    from nvalchemi_toolkit_b200.dynamics import NVTLangevin, _ops

    batch = systems.build(case.system, size, device=device, dtype=dtype)
    model = _build_model(case, device, dtype)
    record: dict[str, Any] = {"name": case.name, "status": "ok", "system": case.system, "size": size,
                              "atoms": batch.num_nodes, "mode": case.mode, "world_size": world,
                              "distributed": case.distributed, "device": str(device), "dtype": case.dtype}
    use_dd = case.distributed or world > 1
    if case.check_forces and use_dd:
        record["force_max_abs_diff"] = force_equivalence(model, batch, case)
        if record["force_max_abs_diff"] > case.force_tolerance:
            record["status"] = "force_mismatch"
            return record
    nc = model.model_config.neighbor_config
    cfg = DomainConfig(cutoff=nc.cutoff if nc is not None else 1.0, skin=case.skin)
    timer = StepTimer(device)
    if case.mode == "forward":
        if use_dd:
            sh = ShardedBatch.from_batch(batch, cfg, model.distribution_spec())
            dm = DistributedModel(model, cfg)
            fn = lambda: dm(sh)  # noqa: E731
        else:
            hooks = model.make_neighbor_hooks()

            def fn() -> Any:
                for h in hooks:
                    h(SimpleNamespace(batch=batch), None)
                return model(batch)
    elif case.mode == "nvt":
        _ops.initialize_velocities(batch.velocities, batch.atomic_masses, case.temperature, batch.batch_idx, random_seed=1)
        if use_dd:
            dyn = NVTLangevin(model, dt=case.dt, temperature=case.temperature, friction=0.01, random_seed=7)
            dp = DomainParallel(dyn, cfg)
            dp.partition(batch)
            dp.compute()
            fn = dp.step
        else:
            dyn = NVTLangevin(model, dt=case.dt, temperature=case.temperature, friction=0.01, random_seed=7,
                              hooks=model.make_neighbor_hooks())
            dyn._call_hooks(type(dyn)._stage_type.BEFORE_COMPUTE, batch)
            dyn.compute(batch)
            fn = lambda: dyn.step(batch)  # noqa: E731
    else:
        raise ValueError(f"unknown mode {case.mode!r}")
    for _ in range(case.warmup):
        fn()
    for _ in range(case.steps):
        with timer:
            fn()
    ms = sorted(timer.samples)
    median = _max_over_ranks(ms[len(ms) // 2], device)
    record.update(ms_per_step_median=median, ms_per_step_min=_max_over_ranks(ms[0], device),
                  atom_steps_per_s=batch.num_nodes / (median * 1e-3))
    return record


def _apply_override(doc: dict, dotted: str, value: str) -> None:
    """``defaults.steps=20`` or ``cases.0.size=8``; values are parsed as YAML scalars."""
    import yaml

    node: Any = doc
    keys = dotted.split(".")
    for k in keys[:-1]:
        node = node[int(k)] if isinstance(node, list) else node.setdefault(k, {})
    last = keys[-1]
    parsed = yaml.safe_load(value)
    if isinstance(node, list):
        node[int(last)] = parsed
    else:
        node[last] = parsed


def load_cases(path: str, overrides: list[str] | None = None) -> list[BenchmarkCase]:
    import yaml

    with open(path, encoding="utf-8") as fh:
        doc = yaml.safe_load(fh)
    for item in overrides or []:
        key, _, value = item.partition("=")
        _apply_override(doc, key, value)
    defaults = doc.get("defaults", {})
    return [BenchmarkCase(**{**defaults, **c}) for c in doc["cases"]]


def run_config(path: str, output: str | None = None, overrides: list[str] | None = None) -> list[dict[str, Any]]:
    results = [run_case(c) for c in load_cases(path, overrides)]
    if output and _world()[0] == 0:
        with open(output, "w", encoding="utf-8") as fh:
            for r in results:
                fh.write(json.dumps(r) + "\n")
    return results


def main(argv: list[str] | None = None) -> int:
    import argparse
    import os

    ap = argparse.ArgumentParser(description="config-driven model-forward / NVT benchmarks")
    ap.add_argument("config")
    ap.add_argument("--output", default=None)
    ap.add_argument("--set", dest="overrides", action="append", default=[], metavar="dotted.key=value",
                    help="override a config entry, e.g. --set defaults.steps=20 --set cases.0.size=8")
    args = ap.parse_args(argv)
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
        backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend)
    for r in run_config(args.config, args.output, args.overrides):
        if _world()[0] == 0:
            print(json.dumps(r))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
