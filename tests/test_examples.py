# SPDX-License-Identifier: Apache-2.0
"""The example scripts run to completion (each in its own interpreter, CPU)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
FAST = ["basic/01_atomic_data_and_batch.py", "basic/02_neighbor_lists.py", "basic/04_batched_fire_relaxation.py",
        "intermediate/06_inflight_batching.py", "intermediate/07_zarr_and_dataloader.py",
        "intermediate/08_train_a_model.py", "advanced/10_ewald_vs_pme.py", "advanced/11_variable_cell_relaxation.py",
        "distributed/12_domain_parallel_md.py", "distributed/14_bring_your_own_mpnn.py",
        "advanced/15_biased_potential.py", "advanced/16_custom_hook_and_convergence.py", "advanced/17_custom_integrator.py",
        "intermediate/18_npt_triclinic.py", "intermediate/19_safety_and_monitoring.py",
        "intermediate/20_sharded_zarr_store.py", "distributed/21_graph_partition.py",
        "distributed/22_relax_then_md_domain_parallel.py", "intermediate/23_data_parallel_training.py",
        "basic/24_nvt_langevin_thermostat.py", "basic/25_ase_interop.py", "advanced/26_mace_nvt.py",
        "advanced/27_learned_charges_plus_ewald.py", "advanced/28_direct_force_model_nve.py",
        "advanced/29_mace_energy_force_training.py", "distributed/30_bring_your_own_graph_transformer.py",
        "distributed/31_npt_domain_parallel.py", "intermediate/32_three_stage_workflow.py",
        "intermediate/33_training_with_live_reporting.py"]
TWO_RANKS = ["distributed/13_stage_pipeline.py", "distributed/30_bring_your_own_graph_transformer.py",
             "distributed/31_npt_domain_parallel.py", "distributed/34_pipeline_monitoring.py"]


@pytest.mark.parametrize("script", FAST)
def test_example_runs(script):
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    env.pop("RANK", None)
    res = subprocess.run([sys.executable, str(ROOT / "examples" / script)], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.strip()


@pytest.mark.parametrize("script", TWO_RANKS)
def test_example_runs_on_two_ranks(script):
    """The distributed examples under ``torchrun`` with two gloo ranks."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    port = 29700 + TWO_RANKS.index(script)
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", str(port), str(ROOT / "examples" / script)], env=env,
                         capture_output=True, text=True, timeout=420)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "rank" in res.stdout
