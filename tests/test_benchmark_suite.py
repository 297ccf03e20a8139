# SPDX-License-Identifier: Apache-2.0
"""Benchmark suite: system builders and the config-driven runners (CPU, tiny sizes)."""
import json

import torch

from nvalchemi_toolkit_b200.benchmark import build, runners, systems


def test_system_builders():
    for name, size, n in (("fcc_cu", 2, 32), ("bcc_fe", 3, 54), ("nacl", 2, 64), ("sio2", 1, 24), ("ch4", 2, 40)):
        b = build(name, size)
        assert b.num_nodes == n and b.atomic_masses.min() > 0 and bool(b.pbc.all())
    b = build("nacl", 2)
    assert abs(float(b.node_charges.sum())) < 1e-6
    s = build("sio2", 1)
    assert abs(float(s.node_charges.sum())) < 1e-5
    d = (s.positions[:8, None] - s.positions[None, 8:]).norm(dim=-1)  # each Si has four O at the bond midpoint distance
    assert int((d < 1.8).sum()) >= 16
    c = build("ar_cluster", 150)
    assert c.num_nodes == 150 and not bool(c.pbc.any())
    assert sorted(systems.SYSTEMS) == ["ar_cluster", "bcc_fe", "ch4", "fcc_cu", "nacl", "sio2", "water"]


def test_runners_from_config(tmp_path):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("""
defaults:
  model: nvalchemi_toolkit_b200.models.lj.LennardJonesModelWrapper
  model_kwargs: {epsilon: 0.0104, sigma: 3.4, cutoff: 6.0, switch_width: 1.0}
  steps: 2
  warmup: 1
  device: cpu
  dtype: float64
cases:
  - {name: fwd, system: fcc_cu, size: 3, mode: forward}
  - {name: nvt, system: fcc_cu, size: 3, mode: nvt}
  - {name: dd, system: fcc_cu, size: 3, mode: nvt, distributed: true, force_tolerance: 1.0e-8}
""")
    res = runners.run_config(str(cfg), str(tmp_path / "out.jsonl"))
    assert [r["status"] for r in res] == ["ok", "ok", "ok"]
    assert res[2]["force_max_abs_diff"] < 1e-8 and res[0]["atoms"] == 108
    rows = [json.loads(l) for l in (tmp_path / "out.jsonl").read_text().splitlines()]
    assert rows[1]["ms_per_step_median"] > 0 and rows[1]["mode"] == "nvt"
    shipped = runners.load_cases(str(__import__("pathlib").Path(runners.__file__).parent / "configs" / "mace_nvt.yaml"))
    assert shipped[0].model.endswith("MACEWrapper") and shipped[2].system == "sio2"


def test_water_box_geometry_and_density():
    import math

    import torch

    from nvalchemi_toolkit_b200.benchmark.systems import water_box

    d = water_box(64, seed=3)
    p = d.positions.double()
    o, h1, h2 = p[0::3], p[1::3], p[2::3]
    assert torch.allclose((h1 - o).norm(dim=1), torch.full((64,), 0.96, dtype=torch.float64), atol=1e-5)
    cosang = ((h1 - o) * (h2 - o)).sum(1) / 0.96 ** 2
    assert torch.allclose(torch.rad2deg(torch.acos(cosang)), torch.full((64,), 104.5, dtype=torch.float64), atol=1e-3)
    vol = float(torch.linalg.det(d.cell.reshape(3, 3).double()))
    assert abs(64 * 18.015 / 0.602214 / vol - 1.0) < 1e-6  # g / cm^3
    assert abs(float(d.charges.sum())) < 1e-5 and d.atomic_numbers.tolist()[:3] == [8, 1, 1]
    oo = torch.cdist(o, o) + 10 * torch.eye(64, dtype=torch.float64)
    assert float(oo.min()) > 1.8 and math.isfinite(vol)


def test_pipeline_benchmark_two_lanes_of_two_stages(tmp_path):
    """Four gloo ranks = two independent lanes of FIRE -> NVT hand-off over water boxes with MACE + D3 + PME; every system
    of the stream reaches the sinks of the MD ranks, lanes terminate independently."""
    import json
    import os
    import subprocess
    import sys

    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
           "--master-port", "29671", "-m", "nvalchemi_toolkit_b200.benchmark.baseline_configs", "pipeline", "--systems", "6",
           "--min-molecules", "5", "--max-molecules", "8", "--relax-steps", "2", "--md-steps", "2", "--channels", "4",
           "--max-atoms", "48", "--max-batch", "2", "--max-neighbors", "48"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["lanes"] == 2 and out["systems_finished"] == 6 and out["unit"] == "atom-steps/s" and out["value"] > 0


import pytest  # noqa: E402


@pytest.mark.gpu
def test_halo_bandwidth_benchmark_single_process_mode():
    """The halo-kernel benchmark in its one-GPU mode (peers are local buffers): every kernel runs, the byte counts follow
    from the arguments and the status word stays clear."""
    import subprocess
    import sys

    out = subprocess.run([sys.executable, "-m", "nvalchemi_toolkit_b200.benchmark.halo_bandwidth", "--single-process", "--rows", "4096",
                          "--owned", "8192", "--peers", "2", "--iters", "3"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["single_process"] and res["world"] == 3 and res["ghost_rows"] == 4096 and res["status"] == 0
    for key, width in (("pull_features_512", 512), ("push_add_features_512", 512), ("pull_add_features_512", 512),
                       ("pull_positions_3", 3), ("push_add_positions_3", 3), ("pull_add_positions_3", 3)):
        assert res[key]["bytes"] == 4096 * width * 4 and res[key]["ms"] > 0 and res[key]["gbs"] > 0
    assert "barrier_us" not in res
