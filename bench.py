# SPDX-License-Identifier: Apache-2.0
"""Headline benchmark: MD atom-steps/s of the 1,048,576-atom fcc-Cu MACE NVT-Langevin configuration.

    python bench.py --gpus N --steps K --warmup W        (torchrun launches one rank per GPU for N > 1)

Prints one JSON line on rank 0.  ``value`` = atoms * K / (device-timed seconds, max over ranks) through the
framework's dynamics engine with all state resident on the device(s); ``e2e`` repeats the measurement with the
state owned by the host: every step copies positions and velocities from pinned host memory, runs one public
``NVTLangevin.step`` and reads the energy, positions and velocities back.
Synthetic data (64^3 conventional cells, a = 3.61 A, 0.05 A noise, 300 K Maxwell-Boltzmann velocities) and
random-initialised weights of the named architecture (2 interactions, 128x0e+128x1o, l_max 3, correlation 3,
8 Bessel functions, 5 A cutoff, fp32 with TF32 tensor-core channel mixes).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "MD atom-steps/s (1,048,576-atom fcc Cu, MACE 2x(128x0e+128x1o) lmax3 corr3, NVT Langevin dt=1fs)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_system(cells: int, device, seed: int = 0, atom_order: str = "lattice"):
    import torch

    from nvalchemi_toolkit_b200 import AtomicData, Batch

    a = 3.61
    g = torch.Generator(device=device).manual_seed(seed)
    base = torch.tensor([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]], device=device)
    r = torch.arange(cells, device=device, dtype=torch.float32)
    grid = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 1, 3)
    pos = ((grid + base[None]).reshape(-1, 3) * a)
    pos = pos + 0.05 * torch.randn(pos.shape, generator=g, device=device)
    if atom_order == "morton":
        from nvalchemi_toolkit_b200.utils.spatial import morton_order

        pos = pos[morton_order(pos, torch.eye(3, device=device) * a * cells, 4.0)].contiguous()
    n = pos.shape[0]
    data = AtomicData.model_construct(
        atomic_numbers=torch.full((n,), 29, dtype=torch.long, device=device), positions=pos,
        atomic_masses=torch.full((n,), 63.546, device=device), velocities=torch.zeros_like(pos),
        forces=torch.zeros_like(pos), energy=torch.zeros(1, 1, device=device),
        cell=(torch.eye(3, device=device) * a * cells).reshape(1, 3, 3),
        pbc=torch.ones(1, 3, dtype=torch.bool, device=device),
        atom_categories=torch.zeros(n, dtype=torch.long, device=device), info={})
    data.model_post_init(None)
    return Batch.from_data_list([data], device=device)


def build_dynamics(device, skin: float, max_neighbors: int):
    import torch

    from nvalchemi_toolkit_b200.dynamics import NVTLangevin
    from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper

    torch.manual_seed(0)
    cfg = MACEConfig(atomic_numbers=[29], r_max=5.0, num_bessel=8, num_polynomial_cutoff=5, max_ell=3,
                     num_interactions=2, channels=128, hidden_lmax=1, correlation=3, avg_num_neighbors=42.0)
    wrapper = MACEWrapper(MACE(cfg).to(device), skin=skin)
    wrapper.eval()
    hooks = wrapper.make_neighbor_hooks(max_neighbors=max_neighbors)
    return NVTLangevin(wrapper, dt=1.0, temperature=300.0, friction=0.01, random_seed=7, hooks=hooks), wrapper


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from nvalchemi_toolkit_b200.dynamics import _ops
    from nvalchemi_toolkit_b200.ops import _native_counter, gemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cells = args.cells
    n_atoms_total = 4 * cells ** 3
    if world > 1:
        from nvalchemi_toolkit_b200.distributed.slab_md import SlabDomainMD

        sim = SlabDomainMD.for_benchmark(cells=cells, device=device, skin=args.skin, max_neighbors=args.max_neighbors,
                                         atom_order=args.atom_order)
        step, sync_energy, e2e_step = sim.step, sim.energy, sim.host_driven_step
        per_rank = torch.tensor(sim.e2e_bytes(), dtype=torch.int64, device=device)
        dist.all_reduce(per_rank)  # bytes of the whole job per step (every rank moves its own atoms)
        counts = tuple(int(x) for x in per_rank.tolist())
        parallelism = f"dd{world} (slabs along x, ghost senders within 5 A cutoff + 1 A skin)"
    else:
        batch = build_system(cells, device, atom_order=args.atom_order)
        dyn, wrapper = build_dynamics(device, args.skin, args.max_neighbors)
        _ops.initialize_velocities(batch.velocities, batch.atomic_masses, 300.0, batch.batch_idx, random_seed=1)
        dyn._call_hooks(type(dyn)._stage_type.BEFORE_COMPUTE, batch)
        dyn.compute(batch)

        def step():
            dyn.step(batch)

        host_pos = torch.empty_like(batch.positions, device="cpu").pin_memory()
        host_vel = torch.empty_like(batch.velocities, device="cpu").pin_memory()
        host_e = torch.empty(1, 1, pin_memory=True)
        host_pos.copy_(batch.positions)
        host_vel.copy_(batch.velocities)

        def e2e_step():
            batch.positions.copy_(host_pos, non_blocking=True)
            batch.velocities.copy_(host_vel, non_blocking=True)
            dyn.step(batch)
            host_pos.copy_(batch.positions, non_blocking=True)
            host_vel.copy_(batch.velocities, non_blocking=True)
            host_e.copy_(batch.energy, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return float(host_e)

        counts = (host_pos.numel() * 4 + host_vel.numel() * 4, host_pos.numel() * 4 + host_vel.numel() * 4 + 4)
        parallelism = "single GPU"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        barrier()
        ms = torch.tensor([t0.elapsed_time(t1)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _native_counter.reset()
    ms = timed(step, args.steps)
    launches = _native_counter.count()
    clocks = sampler.stop() if rank == 0 else {}
    if world > 1 and args.phase_times:
        sim.profile = True
        for _ in range(3):
            step()
        phases = sim.phase_summary()
        sim.profile = False
        if rank == 0:
            print("phase ms:", {k: round(v, 2) for k, v in phases.items()}, "owned", sim.n_owned, "ghost", sim.n_ghost,
                  file=sys.stderr, flush=True)
    for _ in range(min(args.warmup, 2)):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    err = gemm.check_errors(torch.zeros(1, device=device))
    value = n_atoms_total * args.steps / (ms * 1e-3)
    out = {
        "metric": METRIC, "value": value, "unit": "atom-steps/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32 (tf32 tensor-core channel mixes)", "data": "synthetic",
        "config": {"model": "MACE 2 layers 128x0e+128x1o lmax3 corr3 8 Bessel rc=5A (random init)",
                   "global_batch": n_atoms_total, "seq_len": None, "parallelism": parallelism, "atoms": n_atoms_total,
                   "dt_fs": 1.0, "thermostat": "Langevin 300K gamma=0.01/fs", "neighbor_skin_A": args.skin, "atom_order": args.atom_order,
                   "l2_policy": "per-step working set (node features, edge lists) is tens of GB, far larger than the 126 MB L2"},
        "clocks": clocks,
        "e2e": {"value": n_atoms_total * args.steps / (ms_e2e * 1e-3), "unit": "atom-steps/s",
                "h2d_bytes_per_step": counts[0], "d2h_bytes_per_step": counts[1], "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches, "gpu_launches_note": "native operator calls (each launches >= 1 kernel) on rank 0",
        "kernel_error_status": err,
    }
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_reference(args) -> dict:
    """The reference's own code path.  It cannot be installed offline here: its build backend (hatchling) and its
    runtime dependencies (warp, nvalchemiops, tensordict, mace-torch, e3nn, physicsnemo) are not in the wheelhouse."""
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    why = "reference not installable offline: build backend 'hatchling' missing from the wheelhouse; runtime deps " \
          "warp-lang, nvalchemi-toolkit-ops, tensordict, mace-torch, e3nn, nvidia-physicsnemo also absent"
    if os.path.isdir(os.path.join(ref, "nvalchemi")):
        sys.path.insert(0, ref)
        try:
            import nvalchemi  # noqa: F401
            why = "reference imports but its MACE path needs mace-torch/e3nn/nvalchemiops which are absent"
        except Exception as exc:  # pragma: no cover
            why = f"reference import failed: {type(exc).__name__}: {exc}".splitlines()[0]
    return {"impl": "reference", "unavailable": why}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cells", type=int, default=64, help="conventional fcc cells per edge (64 -> 1,048,576 atoms)")
    ap.add_argument("--skin", type=float, default=0.0, help="Verlet skin; 0 rebuilds the list every step (cheaper than the extra edges at this size)")
    ap.add_argument("--max-neighbors", type=int, default=64)
    ap.add_argument("--phase-times", action="store_true", help="multi-GPU: also print per-phase CUDA-event times of rank 0")
    ap.add_argument("--atom-order", default="lattice", choices=["lattice", "morton"],
                    help="memory order of the synthetic atoms: x-major lattice order or a Z-curve over 4 A bins")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(run_reference(args)))
        return
    t = time.time()
    out = run_ours(args)
    if out:
        out["wall_s_total"] = time.time() - t
        print(json.dumps(out))


if __name__ == "__main__":
    main()
