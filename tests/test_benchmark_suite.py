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
    assert sorted(systems.SYSTEMS) == ["ar_cluster", "bcc_fe", "ch4", "fcc_cu", "nacl", "sio2"]


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
