# SPDX-License-Identifier: Apache-2.0
"""Headline benchmark: MD atom-steps/s of the 1,048,576-atom fcc-Cu MACE NVT-Langevin configuration.

    python bench.py --gpus N --steps K --warmup W        (torchrun launches one rank per GPU for N > 1)

Prints one JSON line on rank 0.  ``value`` = atoms * K / (device-timed seconds, max over ranks) of public-API steps:
``NVTLangevin(MACEWrapper).step`` on one GPU, ``DomainParallel(NVTLangevin(MACEWrapper), DomainConfig).step`` on N
(every rank builds the same system and keeps the atoms of its sub-domain; ghost rows travel through peer-mapped memory).
``e2e`` repeats the measurement with the state owned by the host: every step copies positions and velocities from
pinned host memory, runs one step and reads the energy, positions and velocities back.  ``energy_per_atom_step0`` and
``fmax_step0`` do not depend on N when the decomposition is right.  ``baseline`` / ``vs_baseline``: a short run of this
repo's stand-in baseline (N > 1: the same model through ``torch.distributed`` collectives only, also available alone as
``--impl nccl_baseline``; N = 1: the eager-PyTorch statement of the network on a smaller system, per atom).
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


def build_dynamics(device, skin: float, max_neighbors: int, neighbor_hooks: bool = True, backend: str = "auto"):
    import torch

    from nvalchemi_toolkit_b200.dynamics import NVTLangevin
    from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper

    torch.manual_seed(0)
    cfg = MACEConfig(atomic_numbers=[29], r_max=5.0, num_bessel=8, num_polynomial_cutoff=5, max_ell=3,
                     num_interactions=2, channels=128, hidden_lmax=1, correlation=3, avg_num_neighbors=42.0)
    net = MACE(cfg).to(device)
    net.backend = backend
    wrapper = MACEWrapper(net, skin=skin)
    wrapper.eval()
    hooks = wrapper.make_neighbor_hooks(max_neighbors=max_neighbors) if neighbor_hooks else []
    return NVTLangevin(wrapper, dt=1.0, temperature=300.0, friction=0.01, random_seed=7, hooks=hooks), wrapper


class _Job:
    """One configured MD job (single GPU, or domain-decomposed through ``DomainParallel``) with its step functions."""

    def __init__(self, args, device, world: int, peer_memory, halo_width: float | None, cells: int | None = None,
                 backend: str = "auto") -> None:
        import torch
        import torch.distributed as dist

        from nvalchemi_toolkit_b200.dynamics import _ops

        self.world, self.device = world, device
        cells = cells if cells is not None else args.cells
        self.n_atoms = 4 * cells ** 3
        batch = build_system(cells, device, atom_order=args.atom_order)  # the same system on every rank and for every N
        _ops.initialize_velocities(batch.velocities, batch.atomic_masses, 300.0, batch.batch_idx, random_seed=1)
        self.dp = None
        if world > 1:
            from nvalchemi_toolkit_b200.distributed import DomainConfig, DomainParallel

            dyn, self.wrapper = build_dynamics(device, args.skin, args.max_neighbors, neighbor_hooks=False, backend=backend)
            cfg = DomainConfig(cutoff=5.0, skin=args.halo_skin, ghost_width=halo_width, neighbor_skin=args.skin,
                               migration_hysteresis=0.0, peer_memory=peer_memory,
                               grid_dims=tuple(args.grid) if args.grid else None)
            self.dp = DomainParallel(dyn, cfg, max_neighbors=args.max_neighbors)
            self.dp.partition(batch)
            del batch
            self.dp.compute()
            self.dyn = dyn
            self.step = self.dp.step
            grid = self.dp.sharded.partitioner.grid
            mode = "peer-memory NVLink kernels" if getattr(self.dp.model, "engine", None) is not None else \
                "torch.distributed collectives only"
            self.parallelism = f"dd{world} grid {grid[0]}x{grid[1]}x{grid[2]} ({mode})"
        else:
            self.dyn, self.wrapper = build_dynamics(device, args.skin, args.max_neighbors, backend=backend)
            self.batch = batch
            self.dyn._call_hooks(type(self.dyn)._stage_type.BEFORE_COMPUTE, batch)
            self.dyn.compute(batch)
            self.step = lambda: self.dyn.step(batch)
            self.parallelism = "single GPU"
        self._host = None
        self._dist = dist

    @property
    def owned(self):
        return self.dp.sharded.owned if self.dp is not None else self.batch

    def step0_observables(self) -> tuple[float, float, int]:
        """Energy per atom, largest force norm and the largest ghost count of the force evaluation made at set-up."""
        import torch

        b = self.owned
        fmax = b.forces.norm(dim=-1).max().double().reshape(1)
        ghosts = torch.tensor([self.dp.sharded.n_ghost if self.dp is not None else 0], device=self.device)
        if self.world > 1:
            self._dist.all_reduce(fmax, op=self._dist.ReduceOp.MAX)
            self._dist.all_reduce(ghosts, op=self._dist.ReduceOp.MAX)
        return float(b.energy.reshape(-1)[0]) / self.n_atoms, float(fmax), int(ghosts)

    def e2e_bytes(self) -> tuple[int, int]:
        import torch

        n = torch.tensor([self.owned.num_nodes], device=self.device)
        if self.world > 1:
            self._dist.all_reduce(n)
        n = int(n)
        return 2 * n * 12, 2 * n * 12 + 4 * self.world

    def e2e_step(self) -> float:
        """One step with the state owned by the host: positions and velocities of this rank's atoms come from pinned
        host memory, one public ``step`` runs, and positions, velocities and the energy are read back."""
        import torch

        b = self.owned
        n = b.num_nodes
        if self._host is None or self._host[0].shape[0] != n:
            self._host = (torch.empty(n, 3).pin_memory(), torch.empty(n, 3).pin_memory(), torch.empty(1, 1).pin_memory())
            self._host[0].copy_(b.positions)
            self._host[1].copy_(b.velocities)
        hp, hv, he = self._host
        b.positions.copy_(hp, non_blocking=True)
        b.velocities.copy_(hv, non_blocking=True)
        self.step()
        b = self.owned
        if b.num_nodes != n:  # atoms migrated inside the step: the host copy is re-made at the next call
            self._host = None
            torch.cuda.current_stream().synchronize()
            return float(b.energy.reshape(-1)[0])
        hp.copy_(b.positions, non_blocking=True)
        hv.copy_(b.velocities, non_blocking=True)
        he.copy_(b.energy.reshape(1, 1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(he)

    def close(self) -> None:
        import gc

        import torch

        from nvalchemi_toolkit_b200.models.mace import native

        if self.dp is not None:
            self.dp.close()
        self.dp = self.dyn = self.wrapper = self.step = self._host = None
        if hasattr(self, "batch"):
            del self.batch
        native.release_radial_cache()
        gc.collect()
        torch.cuda.empty_cache()


def run_ours(args, impl: str = "ours") -> dict:
    import torch
    import torch.distributed as dist

    from nvalchemi_toolkit_b200.models.mace import native
    from nvalchemi_toolkit_b200.ops import _native_counter, gemm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

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

    def measure(job, steps, warmup):
        for _ in range(warmup):
            job.step()
        return timed(job.step, steps)

    peer = None if impl == "ours" else False
    job = _Job(args, device, world, peer, args.halo_width)
    n_atoms_total = job.n_atoms
    e_atom, fmax0, n_ghost = job.step0_observables()
    for _ in range(args.warmup):
        job.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    _native_counter.reset()
    ms = timed(job.step, args.steps)
    launches = _native_counter.count()
    clocks = sampler.stop() if rank == 0 else {}
    cache_active = bool(native._h3_pool)
    for _ in range(min(args.warmup, 2)):
        job.e2e_step()
    ms_e2e = timed(job.e2e_step, args.steps)
    counts = job.e2e_bytes()
    err = gemm.check_errors(torch.zeros(1, device=device))
    engine = getattr(job.dp.model, "engine", None) if job.dp is not None else None
    peer_status = engine.status() if engine is not None else 0
    phases = None
    if args.phase_times and engine is not None:  # separate, untimed steps: the event records are not in the headline
        engine.phase_events = []
        for _ in range(max(3, min(args.steps, 5))):
            job.step()
        phases = {k: round(v, 3) for k, v in engine.phase_times_ms().items()}
        engine.phase_events = None
    rebuilds = job.dp.num_rebuilds if job.dp is not None else 0
    parallelism = job.parallelism
    value = n_atoms_total * args.steps / (ms * 1e-3)
    job.close()

    extra: dict = {}
    if impl == "ours" and world > 1 and args.alt_halo_width and args.alt_halo_width != args.halo_width:
        alt = _Job(args, device, world, None, args.alt_halo_width)
        _, _, alt_ghost = alt.step0_observables()
        k = max(3, min(args.steps, 5))
        alt_ms = measure(alt, k, 3)
        extra["alt_halo"] = {"halo_width_A": args.alt_halo_width, "n_ghost_max": alt_ghost,
                             "value": n_atoms_total * k / (alt_ms * 1e-3), "ms_per_step": alt_ms / k, "steps": k}
        alt.close()
    baseline = None
    if impl == "ours" and args.baseline_steps > 0:
        try:
            baseline = _baseline_arm(args, device, world, measure, n_atoms_total)
        except Exception as exc:  # the stand-in arm must not take the measurement down with it
            baseline = None
            extra["baseline_error"] = f"{type(exc).__name__}: {exc}".splitlines()[0][:300]
            if world > 1:
                raise
    if phases is not None:
        extra["phase_ms_rank0"] = phases
    out = _result(locals())
    out.update(extra)
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def _baseline_arm(args, device, world, measure, n_atoms_total) -> dict:
    k = args.baseline_steps
    if world > 1:
        # the same model and system through the generic layer: torch.distributed collectives only, ghost layer two
        # cutoffs deep (no peer-memory kernels); the repo's own stand-in for a library-collective build
        base = _Job(args, device, world, False, None)
        b_ms = measure(base, k, 3)
        baseline = {"impl": "nccl_baseline", "value": n_atoms_total * k / (b_ms * 1e-3), "ms_per_step": b_ms / k,
                    "steps": k, "atoms": n_atoms_total,
                    "note": "this repo's native MACE under the generic DomainParallel route: NCCL all-to-all halo, "
                            "2-cutoff ghost layer recomputed, reverse halo for forces"}
    else:
        # no communication on one GPU: the stand-in is the plain-PyTorch (eager, autograd) statement of the same
        # network on a system small enough for its edge tensors, compared per atom
        base = _Job(args, device, 1, False, None, cells=args.baseline_cells, backend="torch")
        b_ms = measure(base, k, 3)
        baseline = {"impl": "torch_eager_restatement", "value": base.n_atoms * k / (b_ms * 1e-3),
                    "ms_per_step": b_ms / k, "steps": k, "atoms": base.n_atoms,
                    "note": "same architecture and weights in eager PyTorch with autograd forces; smaller system "
                            "(its per-edge tensors do not fit at 1M atoms); per-atom throughput"}
    base.close()
    return baseline


def _result(v: dict) -> dict:
    args, value, baseline, ms, ms_e2e, counts = v["args"], v["value"], v["baseline"], v["ms"], v["ms_e2e"], v["counts"]
    n_atoms_total, world = v["n_atoms_total"], v["world"]
    return {
        "metric": METRIC, "value": value, "unit": "atom-steps/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (value / baseline["value"]) if baseline else None,
        "dtype": "fp32 (tf32 tensor-core channel mixes)", "data": "synthetic", "impl": v["impl"],
        "config": {"model": "MACE 2 layers 128x0e+128x1o lmax3 corr3 8 Bessel rc=5A (random init)",
                   "global_batch": n_atoms_total, "seq_len": None, "parallelism": v["parallelism"], "atoms": n_atoms_total,
                   "dt_fs": 1.0, "thermostat": "Langevin 300K gamma=0.01/fs", "neighbor_skin_A": args.skin,
                   "atom_order": args.atom_order, "halo_width_A": args.halo_width if world > 1 else None,
                   "halo_skin_A": args.halo_skin if world > 1 else None, "n_ghost_max": v["n_ghost"],
                   "radial_cache_active": v["cache_active"], "ghost_rebuilds": v["rebuilds"],
                   "l2_policy": "per-step working set (node features, edge lists) is tens of GB, far larger than the 126 MB L2"},
        "energy_per_atom_step0": v["e_atom"], "fmax_step0": v["fmax0"],
        "clocks": v["clocks"],
        "e2e": {"value": n_atoms_total * args.steps / (ms_e2e * 1e-3), "unit": "atom-steps/s",
                "h2d_bytes_per_step": counts[0], "d2h_bytes_per_step": counts[1], "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": v["launches"], "gpu_launches_note": "native operator calls (each launches >= 1 kernel) on rank 0",
        "kernel_error_status": v["err"], "peer_status": v["peer_status"], "baseline": baseline,
    }


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
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_baseline"],
                    help="ours; the unmodified reference (unavailable offline); or this repo's model through the generic "
                         "domain layer with torch.distributed collectives only")
    ap.add_argument("--cells", type=int, default=64, help="conventional fcc cells per edge (64 -> 1,048,576 atoms)")
    ap.add_argument("--skin", type=float, default=0.0, help="Verlet skin; 0 rebuilds the list every step (cheaper than the extra edges at this size)")
    ap.add_argument("--max-neighbors", type=int, default=64)
    ap.add_argument("--halo-width", type=float, default=10.0, help="ghost layer depth in A (multi-GPU)")
    ap.add_argument("--alt-halo-width", type=float, default=6.0,
                    help="a second, short measurement at this ghost depth (multi-GPU; 0 disables it)")
    ap.add_argument("--halo-skin", type=float, default=1.0, help="ghost lists are rebuilt when an atom moved half of this")
    ap.add_argument("--grid", type=int, nargs=3, default=None, help="rank grid (default: least cut surface)")
    ap.add_argument("--baseline-steps", type=int, default=3, help="timed steps of the stand-in baseline arm (0: skip)")
    ap.add_argument("--baseline-cells", type=int, default=14, help="cells per edge of the single-GPU eager-PyTorch arm")
    ap.add_argument("--phase-times", action="store_true",
                    help="multi-GPU: after the timed steps, CUDA-event times of the phases of a few extra steps (rank 0)")
    ap.add_argument("--atom-order", default="lattice", choices=["lattice", "morton"],
                    help="memory order of the synthetic atoms: x-major lattice order or a Z-curve over 4 A bins")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(run_reference(args)))
        return
    t = time.time()
    out = run_ours(args, args.impl)
    if out:
        out["wall_s_total"] = time.time() - t
        print(json.dumps(out))


if __name__ == "__main__":
    main()
