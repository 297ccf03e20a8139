# SPDX-License-Identifier: Apache-2.0
"""Runners for the relaxation and training workloads next to the headline MD benchmark: synthetic data of the named
shapes, random-initialised weights of the named MACE architecture, one JSON line per run.

    python -m nvalchemi_toolkit_b200.benchmark.baseline_configs relax --systems 512
    python -m nvalchemi_toolkit_b200.benchmark.baseline_configs train --structures 512 --steps 8
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m \\
        nvalchemi_toolkit_b200.benchmark.baseline_configs train ...      (data parallel: fused gradient all-reduce)
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m \\
        nvalchemi_toolkit_b200.benchmark.baseline_configs pipeline       (4 FIRE ranks | 4 NVT ranks, water + D3 + PME)

``relax``: FIRE to ``fmax`` with inflight batching (``SizeAwareSampler`` refills the slots of converged systems) over a
stream of periodic fcc / bcc supercells of 32-256 atoms of Cu, Ni, Al, Fe with lattice constants 2.8-4.1 A and 0.1 A
noise; with N ranks every rank relaxes its share of the stream.  Metric: relaxed systems per second (whole job).
``train``: Adam (lr 1e-3) on ``energy MSE + 100 * force MSE`` with 64 structures per rank and step; fcc Cu supercells of
64-216 atoms with 0.15 A displacements labelled by a Lennard-Jones potential (eps 0.4 eV, sigma 2.34 A, 6 A cutoff).
Metric: structures per second (whole job).  Both follow the reference's timing convention: warm-up, then device-timed
steps, maximum over ranks (``benchmark/distributed/_benchmark_common.py:1341-1474``)."""
from __future__ import annotations

import argparse
import json
import os
import time
from typing import Any

import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200.benchmark import systems


def _mace(device: torch.device, species: list[int], backend: str = "auto") -> Any:
    from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper

    torch.manual_seed(0)
    cfg = MACEConfig(atomic_numbers=species, r_max=5.0, num_bessel=8, num_polynomial_cutoff=5, max_ell=3,
                     num_interactions=2, channels=128, hidden_lmax=1, correlation=3, avg_num_neighbors=40.0)
    net = MACE(cfg, backend=backend).to(device)
    return MACEWrapper(net)


def _dist() -> tuple[int, int, torch.device]:
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", **({"device_id": device} if device.type == "cuda" else {}))
    return rank, world, device


def _max_over_ranks(seconds: float, device: torch.device, world: int) -> float:
    if world == 1:
        return seconds
    t = torch.tensor([seconds], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


class SupercellStream:
    """Dataset protocol of ``SizeAwareSampler`` over synthetic metal supercells (generated on first access)."""

    _SPEC = {29: ("fcc", 3.61), 28: ("fcc", 3.52), 13: ("fcc", 4.05), 26: ("bcc", 2.87)}

    def __init__(self, n: int, seed: int = 0, offset: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        self.z = [list(self._SPEC)[int(i)] for i in torch.randint(0, 4, (n + offset,), generator=g)][offset:]
        self.scale = (0.95 + 0.1 * torch.rand(n + offset, generator=g))[offset:].tolist()
        self.reps = torch.randint(2, 5, (n + offset,), generator=g)[offset:].tolist()  # fcc 32..256 atoms, bcc 16..128
        self.seed = seed + offset
        self._cache: dict[int, Any] = {}

    def __len__(self) -> int:
        return len(self.z)

    def _atoms(self, i: int) -> int:
        kind, _ = self._SPEC[self.z[i]]
        reps = self.reps[i] if kind == "fcc" else self.reps[i] + 1
        return (4 if kind == "fcc" else 2) * reps ** 3

    def get_metadata(self, i: int) -> tuple[int, int]:
        return self._atoms(i), 0

    def __getitem__(self, i: int) -> tuple[Any, dict]:
        if i not in self._cache:
            kind, a = self._SPEC[self.z[i]]
            a = min(max(a * self.scale[i], 2.8), 4.1)
            if kind == "fcc":
                d = systems.fcc(self.reps[i], a=a, z=self.z[i], noise=0.1, seed=self.seed + i)
            else:
                d = systems.bcc_iron(self.reps[i] + 1, a=a, noise=0.1, seed=self.seed + i)
            d.__dict__["velocities"] = torch.zeros_like(d.positions)
            self._cache[i] = d
        return self._cache[i], {}


def relax(args: argparse.Namespace) -> dict:
    from nvalchemi_toolkit_b200.dynamics import FIRE, ConvergenceHook, FusedStage, HostMemory, SizeAwareSampler

    rank, world, device = _dist()
    share = args.systems // world
    data = SupercellStream(share, seed=1, offset=rank * share)
    wrapper = _mace(device, [13, 26, 28, 29]).eval()

    def workflow(stream: Any, capacity: int) -> tuple[Any, Any]:
        sampler = SizeAwareSampler(stream, max_atoms=args.max_atoms, max_batch_size=args.max_batch)
        sink = HostMemory(capacity=capacity)
        fire = FIRE(wrapper, dt=args.dt, convergence_hook=ConvergenceHook.from_fmax(args.fmax),
                    hooks=wrapper.make_neighbor_hooks(max_neighbors=args.max_neighbors))
        return FusedStage(sub_stages=[(0, fire)], sampler=sampler, sinks=[sink], refill_frequency=args.refill_frequency,
                          device_type=device.type), sink

    # untimed: the stream is materialised in host memory (the timed region measures relaxation, not the synthetic data
    # generator) and a short relaxation of a separate small stream warms up allocator pools, lazily built weight packs and
    # first-use library initialisation
    for i in range(len(data)):
        data[i]
    if args.warmup_systems > 0:
        warm, _ = workflow(SupercellStream(min(args.warmup_systems, share), seed=99), args.warmup_systems)
        warm.run(n_steps=args.max_steps)
    flow, sink = workflow(data, share)
    if device.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    flow.run(n_steps=args.max_steps)
    if device.type == "cuda":
        torch.cuda.synchronize()
    seconds = _max_over_ranks(time.perf_counter() - t0, device, world)
    done = sink.read()
    n_done = torch.tensor([0 if done is None else done.num_graphs, 0 if done is None else done.num_nodes], device=device)
    if world > 1:
        dist.all_reduce(n_done)
    return {"metric": "FIRE relaxations/s with inflight batching (MACE 2x(128x0e+128x1o) lmax3 corr3, fmax %.3g eV/A)" % args.fmax,
            "value": int(n_done[0]) / seconds, "unit": "systems/s", "n_gpus": world, "systems_relaxed": int(n_done[0]),
            "systems_in_stream": share * world, "atoms_relaxed": int(n_done[1]), "fused_steps_rank0": flow.step_count,
            "seconds": seconds, "data": "synthetic", "config": {"max_atoms": args.max_atoms, "max_batch": args.max_batch,
                                                               "dt": args.dt, "refill_frequency": args.refill_frequency}}


def _lj_labels(batch: Any, eps: float = 0.4, sigma: float = 2.34, cutoff: float = 6.0) -> None:
    """Energies and forces of a Lennard-Jones teacher written into the batch (float64 on the batch's device)."""
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
    from nvalchemi_toolkit_b200.neighbors import compute_neighbors

    teacher = LennardJonesModelWrapper(epsilon=eps, sigma=sigma, cutoff=cutoff, switch_width=0.5)
    teacher.model_config.active_outputs = {"energy", "forces"}
    compute_neighbors(batch, config=teacher.model_config.neighbor_config)
    out = teacher(batch)
    batch["energy"] = out["energy"].detach().reshape(batch.num_graphs, 1).clone()
    batch["forces"] = out["forces"].detach().clone()


def train(args: argparse.Namespace) -> dict:
    from nvalchemi_toolkit_b200 import Batch
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage  # noqa: F401  (neighbour hooks live on the wrapper)
    from nvalchemi_toolkit_b200.neighbors import compute_neighbors
    from nvalchemi_toolkit_b200.training import EnergyMSELoss, ForceMSELoss, OptimizerConfig, TrainingStrategy
    from nvalchemi_toolkit_b200.training.hooks.library import FusedGradAllReduceHook, GradientAccumulationHook

    rank, world, device = _dist()
    micro = args.micro_batch or args.batch
    if args.batch % micro:
        raise SystemExit("train: --batch must be a multiple of --micro-batch")
    accumulate = args.batch // micro
    per_rank = args.structures // world
    g = torch.Generator().manual_seed(7 + rank)
    reps = torch.randint(0, 3, (per_rank,), generator=g).tolist()
    shapes = [(2, 2, 4), (3, 3, 4), (3, 3, 6)]  # 64, 144, 216 atoms
    wrapper = _mace(device, [29], backend="torch" if args.backend == "torch" else "auto")
    wrapper.train()
    nc = wrapper.model_config.neighbor_config
    loader = []
    for i in range(0, per_rank, micro):
        items = []
        for k in range(i, min(i + micro, per_rank)):
            rx, ry, rz = shapes[reps[k]]
            items.append(systems._crystal(torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]]),
                                          torch.full((4,), 29), 3.61, (rx, ry, rz), 0.15, 1000 * rank + k, torch.float32))
        b = Batch.from_data_list(items, device=device)
        _lj_labels(b)
        compute_neighbors(b, config=nc)  # the student's own (5 A) list replaces the teacher's
        loader.append(b)
    hooks = ([GradientAccumulationHook(steps=accumulate)] if accumulate > 1 else []) + ([FusedGradAllReduceHook()] if world > 1 else [])
    loss = EnergyMSELoss(weight=1.0) + ForceMSELoss(weight=100.0)
    st = TrainingStrategy(wrapper, OptimizerConfig(kwargs={"lr": 1e-3}), loss_fn=loss, num_steps=args.warmup, devices=[str(device)],
                          hooks=hooks)
    st.run(loader)  # warm-up steps (allocator, autotuned library kernels)
    if device.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    st.num_steps = args.warmup + args.steps
    t0 = time.perf_counter()
    st.run(loader)
    if device.type == "cuda":
        torch.cuda.synchronize()
    seconds = _max_over_ranks(time.perf_counter() - t0, device, world)
    n_struct = args.steps * args.batch * world
    return {"metric": "MLIP training structures/s (MACE 2x(128x0e+128x1o), Adam, energy + 100 x force MSE, batch %d / rank)" % args.batch,
            "value": n_struct / seconds, "unit": "structures/s", "n_gpus": world, "steps": args.steps, "seconds": seconds,
            "last_loss": float(st.last_losses["total_loss"]), "backend": args.backend, "data": "synthetic (LJ-labelled fcc Cu)",
            "micro_batch": micro, "accumulation_steps": accumulate,
            "gradient_allreduce": "fused peer-memory all-reduce" if world > 1 and device.type == "cuda" else "none"}


class WaterStream:
    """Dataset protocol of ``SizeAwareSampler`` over periodic water boxes of ``lo``-``hi`` molecules (3 atoms each)."""

    def __init__(self, n: int, lo: int = 512, hi: int = 1024, seed: int = 0, offset: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        self.molecules = torch.randint(lo, hi + 1, (n + offset,), generator=g)[offset:].tolist()
        self.seed = seed + offset
        self._cache: dict[int, Any] = {}

    def __len__(self) -> int:
        return len(self.molecules)

    def get_metadata(self, i: int) -> tuple[int, int]:
        return 3 * self.molecules[i], 0

    def __getitem__(self, i: int) -> tuple[Any, dict]:
        if i not in self._cache:
            self._cache[i] = systems.water_box(self.molecules[i], seed=self.seed + i)
        return self._cache[i], {}


def _water_model(device: torch.device, channels: int) -> Any:
    """MACE (2 layers, ``channels`` x (0e + 1o), lmax 3, correlation 3, 5 A) + DFT-D3(BJ) + PME (alpha 0.3 / A, 1 A mesh)."""
    from nvalchemi_toolkit_b200.models.dftd3 import DFTD3ModelWrapper, DFTD3Parameters
    from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper
    from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper
    from nvalchemi_toolkit_b200.models.pipeline import PipelineGroup, PipelineModelWrapper

    torch.manual_seed(0)
    cfg = MACEConfig(atomic_numbers=[1, 8], r_max=5.0, num_bessel=8, num_polynomial_cutoff=5, max_ell=3, num_interactions=2,
                     channels=channels, hidden_lmax=1, correlation=3, avg_num_neighbors=50.0)
    mace = MACEWrapper(MACE(cfg, backend="auto").to(device)).eval()
    d3 = DFTD3ModelWrapper("pbe", parameters=DFTD3Parameters.synthetic(10), cutoff=10.0)  # synthetic reference tables
    pme = PMEModelWrapper(cutoff=9.0, alpha=0.3, mesh_spacing=1.0, charge_key="charges")
    model = PipelineModelWrapper([PipelineGroup([mace]), PipelineGroup([d3]), PipelineGroup([pme])])
    model.model_config.active_outputs = {"energy", "forces"}
    return model.to(device)


def pipeline(args: argparse.Namespace) -> dict:
    """Relaxation ranks feed MD ranks: ``world / 2`` lanes, lane ``l`` = FIRE on rank ``l`` handing each system after
    ``--relax-steps`` iterations to NVT-Langevin on rank ``l + world / 2`` (``--md-steps`` steps), inflight batching on the
    first stage, hand-off over ``torch.distributed`` point-to-point.  One rank runs both stages fused on its GPU."""
    from nvalchemi_toolkit_b200.dynamics import FIRE, FusedStage, HostMemory, NVTLangevin, SizeAwareSampler
    from nvalchemi_toolkit_b200.dynamics.pipeline import DistributedPipeline

    rank, world, device = _dist()
    if world > 1 and world % 2:
        raise SystemExit("pipeline: the number of ranks must be 1 or even (half relax, half run MD)")
    lanes = max(1, world // 2)
    lane = rank % lanes
    share = args.systems // lanes
    model = _water_model(device, args.channels)
    hooks = lambda: model.make_neighbor_hooks(max_neighbors=args.max_neighbors)  # noqa: E731
    data = WaterStream(share, args.min_molecules, args.max_molecules, seed=2, offset=lane * share)
    sampler = SizeAwareSampler(data, max_atoms=args.max_atoms, max_batch_size=args.max_batch)
    sink = HostMemory(capacity=share)
    fire = FIRE(model, dt=args.dt_relax, n_steps=args.relax_steps, hooks=hooks(), sampler=sampler, device_type=device.type,
                max_batch_size=args.max_batch)
    md = NVTLangevin(model, dt=args.dt_md, temperature=300.0, friction=0.01, random_seed=7, n_steps=args.md_steps,
                     hooks=hooks(), sinks=[sink], device_type=device.type, max_batch_size=2 * args.max_batch)
    if world == 1:
        flow: Any = FusedStage(sub_stages=[(0, fire), (1, md)], sampler=sampler, sinks=[sink], refill_frequency=1,
                               device_type=device.type)
        run = lambda: flow.run(n_steps=args.max_iterations)  # noqa: E731
    else:
        groups = [dist.new_group([ln, ln + lanes]) for ln in range(lanes)]  # created by every rank, in the same order
        flow = DistributedPipeline({lane: fire, lane + lanes: md}, group=groups[lane])
        flow.setup()
        run = lambda: flow.run(max_iterations=args.max_iterations)  # noqa: E731
    if device.type == "cuda":
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    run()
    if device.type == "cuda":
        torch.cuda.synchronize()
    seconds = _max_over_ranks(time.perf_counter() - t0, device, world)
    done = sink.read()
    n_done = torch.tensor([0 if done is None else done.num_graphs, 0 if done is None else done.num_nodes], device=device)
    if world > 1:
        dist.all_reduce(n_done)
    steps_per_atom = args.relax_steps + args.md_steps
    return {"metric": "two-stage pipeline (FIRE ranks | NVT-Langevin ranks), water boxes, MACE + DFT-D3(BJ) + PME",
            "value": int(n_done[1]) * steps_per_atom / seconds, "unit": "atom-steps/s", "systems_per_s": int(n_done[0]) / seconds,
            "n_gpus": world, "lanes": lanes, "systems_finished": int(n_done[0]), "systems_in_stream": share * lanes,
            "atoms_finished": int(n_done[1]), "seconds": seconds, "data": "synthetic (water boxes, 1.0 g/cm^3)",
            "config": {"relax_steps": args.relax_steps, "md_steps": args.md_steps, "molecules": [args.min_molecules, args.max_molecules],
                       "max_atoms": args.max_atoms, "max_batch": args.max_batch, "channels": args.channels,
                       "d3": "BJ damping, synthetic reference tables", "pme": "alpha 0.3 / A, 1 A mesh, order 5"}}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("relax")
    r.add_argument("--systems", type=int, default=4096)
    r.add_argument("--max-atoms", type=int, default=16384)
    r.add_argument("--max-batch", type=int, default=128)
    r.add_argument("--max-neighbors", type=int, default=96)
    r.add_argument("--fmax", type=float, default=0.05)
    r.add_argument("--dt", type=float, default=0.1)
    r.add_argument("--refill-frequency", type=int, default=5)
    r.add_argument("--max-steps", type=int, default=None)
    r.add_argument("--warmup-systems", type=int, default=128, help="systems of the untimed warm-up relaxation (0: none)")
    t = sub.add_parser("train")
    t.add_argument("--structures", type=int, default=1024, help="size of the synthetic training set (whole job)")
    t.add_argument("--batch", type=int, default=8,
                   help="structures per rank and step (the differentiable PyTorch path keeps every per-edge tensor for the "
                        "double backward: 64 structures of this size need more than 180 GB)")
    t.add_argument("--micro-batch", type=int, default=None,
                   help="structures per forward / backward pass; gradients of batch / micro-batch passes are accumulated "
                        "before the (single) reduction and optimiser step, e.g. --batch 64 --micro-batch 8")
    t.add_argument("--steps", type=int, default=8, help="optimiser steps in the timed region")
    t.add_argument("--warmup", type=int, default=2)
    t.add_argument("--backend", default="torch", choices=["torch"], help="differentiable path used under autograd")
    pl = sub.add_parser("pipeline")
    pl.add_argument("--systems", type=int, default=64, help="water boxes in the stream (whole job)")
    pl.add_argument("--min-molecules", type=int, default=512)
    pl.add_argument("--max-molecules", type=int, default=1024)
    pl.add_argument("--relax-steps", type=int, default=20)
    pl.add_argument("--md-steps", type=int, default=20)
    pl.add_argument("--max-atoms", type=int, default=16384)
    pl.add_argument("--max-batch", type=int, default=6)
    pl.add_argument("--max-neighbors", type=int, default=512)
    pl.add_argument("--channels", type=int, default=128)
    pl.add_argument("--dt-relax", type=float, default=0.05)
    pl.add_argument("--dt-md", type=float, default=0.5)
    pl.add_argument("--max-iterations", type=int, default=None)
    args = ap.parse_args(argv)
    out = {"relax": relax, "train": train, "pipeline": pipeline}[args.cmd](args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
