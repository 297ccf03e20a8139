# SPDX-License-Identifier: Apache-2.0
"""Runners for the relaxation and training workloads next to the headline MD benchmark: synthetic data of the named
shapes, random-initialised weights of the named MACE architecture, one JSON line per run.

    python -m nvalchemi_toolkit_b200.benchmark.baseline_configs relax --systems 512
    python -m nvalchemi_toolkit_b200.benchmark.baseline_configs train --structures 512 --steps 8
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m \\
        nvalchemi_toolkit_b200.benchmark.baseline_configs train ...      (data parallel: fused gradient all-reduce)

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
    sampler = SizeAwareSampler(data, max_atoms=args.max_atoms, max_batch_size=args.max_batch)
    sink = HostMemory(capacity=share)
    fire = FIRE(wrapper, dt=args.dt, convergence_hook=ConvergenceHook.from_fmax(args.fmax),
                hooks=wrapper.make_neighbor_hooks(max_neighbors=args.max_neighbors))
    flow = FusedStage(sub_stages=[(0, fire)], sampler=sampler, sinks=[sink], refill_frequency=args.refill_frequency,
                      device_type=device.type)
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
    from nvalchemi_toolkit_b200.training.hooks.library import FusedGradAllReduceHook

    rank, world, device = _dist()
    per_rank = args.structures // world
    g = torch.Generator().manual_seed(7 + rank)
    reps = torch.randint(0, 3, (per_rank,), generator=g).tolist()
    shapes = [(2, 2, 4), (3, 3, 4), (3, 3, 6)]  # 64, 144, 216 atoms
    wrapper = _mace(device, [29], backend="torch" if args.backend == "torch" else "auto")
    wrapper.train()
    nc = wrapper.model_config.neighbor_config
    loader = []
    for i in range(0, per_rank, args.batch):
        items = []
        for k in range(i, min(i + args.batch, per_rank)):
            rx, ry, rz = shapes[reps[k]]
            items.append(systems._crystal(torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]]),
                                          torch.full((4,), 29), 3.61, (rx, ry, rz), 0.15, 1000 * rank + k, torch.float32))
        b = Batch.from_data_list(items, device=device)
        _lj_labels(b)
        compute_neighbors(b, config=nc)  # the student's own (5 A) list replaces the teacher's
        loader.append(b)
    hooks = [FusedGradAllReduceHook()] if world > 1 else []
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
            "gradient_allreduce": "fused peer-memory all-reduce" if world > 1 and device.type == "cuda" else "none"}


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
    t = sub.add_parser("train")
    t.add_argument("--structures", type=int, default=1024, help="size of the synthetic training set (whole job)")
    t.add_argument("--batch", type=int, default=8,
                   help="structures per rank and step (the differentiable PyTorch path keeps every per-edge tensor for the "
                        "double backward: 64 structures of this size need more than 180 GB)")
    t.add_argument("--steps", type=int, default=8)
    t.add_argument("--warmup", type=int, default=2)
    t.add_argument("--backend", default="torch", choices=["torch"], help="differentiable path used under autograd")
    args = ap.parse_args(argv)
    out = relax(args) if args.cmd == "relax" else train(args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
