# SPDX-License-Identifier: Apache-2.0
"""Bounds-checked debug mode: bad index arguments are caught on the host, before a kernel sees them; a full model
evaluation and a dynamics step pass with every operator call validated."""
import pytest
import torch

from nvalchemi_toolkit_b200.ops import _native, debug_bounds
from nvalchemi_toolkit_b200.ops._native_counter import ops

from tests.helpers import fcc_supercell

pytestmark = pytest.mark.skipif(not _native.available(), reason="native library not built")


@pytest.fixture()
def checked():
    debug_bounds.enable(True)
    yield
    debug_bounds.enable(False)


def test_bad_batch_index_and_rows_are_reported(checked, device):
    v = torch.zeros(4, 3, device=device)
    m = torch.ones(4, device=device)
    bad = torch.tensor([0, 1, 2, 1], dtype=torch.int32, device=device)
    with pytest.raises(IndexError, match=r"compute_kinetic_energy.*batch_idx.*outside \[0, 2\)"):
        ops.compute_kinetic_energy(v, m, bad, 2)
    with pytest.raises(IndexError, match="batch_idx.*below the lower bound"):
        ops.compute_kinetic_energy(v, m, torch.tensor([0, -1, 0, 0], dtype=torch.int32, device=device), 2)
    with pytest.raises(IndexError, match="batch_idx.*3 entries for 4 rows"):
        ops.vv_velocity_finalize(v, v.clone(), m, torch.ones(2, device=device), bad[:3])
    src, dst = torch.zeros(3, 2, device=device), torch.zeros(5, 2, device=device)
    with pytest.raises(IndexError, match="copy_rows.*src_rows"):
        ops.copy_rows(src, torch.tensor([0, 3], device=device), dst, torch.tensor([0, 1], device=device))
    with pytest.raises(IndexError, match="not non-decreasing"):
        ops.segmented_copy_planned(src, torch.tensor([0, 2, 1], dtype=torch.int32, device=device),
                                   torch.tensor([0, 2], dtype=torch.int32, device=device), dst)
    with pytest.raises(IndexError, match="past the 5 rows of the destination"):
        ops.segmented_copy_planned(src, torch.tensor([0, 2, 3], dtype=torch.int32, device=device),
                                   torch.tensor([-1, 5], dtype=torch.int32, device=device), dst)
    ok = ops.compute_kinetic_energy(v, m, torch.tensor([0, 1, 1, 0], dtype=torch.int32, device=device), 2)
    assert ok.shape == (2,)


def test_model_and_dynamics_step_pass_under_validation(checked, device):
    """A MACE evaluation (native kernels on the GPU) and an NVE step with neighbour-list rebuild run clean with every
    operator call validated, and calls were in fact validated."""
    from nvalchemi_toolkit_b200.data.batch import Batch
    from nvalchemi_toolkit_b200.dynamics import NVE
    from nvalchemi_toolkit_b200.dynamics.base import DynamicsStage
    from nvalchemi_toolkit_b200.hooks.neighbor_list import NeighborListHook
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

    before = debug_bounds.num_checked
    batch = Batch.from_data_list([fcc_supercell(3, a=5.26, z=18), fcc_supercell(3, a=5.3, z=18, seed=1)], device=device)
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=8.0)
    dyn = NVE(model, dt=1.0, n_steps=3,
              hooks=[NeighborListHook(model.model_config.neighbor_config, stage=DynamicsStage.BEFORE_COMPUTE)])
    dyn.run(batch)
    assert debug_bounds.num_checked > before + 5
    assert torch.isfinite(batch.positions).all()


@pytest.mark.gpu
def test_native_mace_evaluation_passes_under_validation(checked):
    """Every native operator call of a MACE energy / force / stress evaluation (CSR build, radial MLP, fused convolutions,
    grouped GEMMs, symmetric contraction, readout) has in-range index arguments."""
    from nvalchemi_toolkit_b200.data.batch import Batch
    from nvalchemi_toolkit_b200.models.mace import MACE, MACEConfig, MACEWrapper
    from nvalchemi_toolkit_b200.neighbors import compute_neighbors

    torch.manual_seed(3)
    model = MACE(MACEConfig(atomic_numbers=[29, 28], channels=32, avg_num_neighbors=40.0), backend="native").cuda()
    b = Batch.from_data_list([fcc_supercell(3, noise=0.1), fcc_supercell(2, a=3.9, noise=0.1, seed=7)], device="cuda")
    w = MACEWrapper(model).eval()
    w.model_config.active_outputs = {"energy", "forces", "stress"}
    compute_neighbors(b, config=w.model_config.neighbor_config)
    before = debug_bounds.num_checked
    out = w(b)
    assert debug_bounds.num_checked > before + 10
    assert torch.isfinite(out["forces"]).all()
