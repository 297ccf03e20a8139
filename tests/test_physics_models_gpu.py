# SPDX-License-Identifier: Apache-2.0
"""CUDA runs of the electrostatics and dispersion kernels against float64 CPU results of the same models, and the
generic domain-decomposition layer on one GPU (periodic self-images)."""
from types import SimpleNamespace

import pytest
import torch

from nvalchemi_toolkit_b200 import Batch

pytestmark = pytest.mark.gpu


def _run(model, batch):
    for h in model.make_neighbor_hooks():
        h(SimpleNamespace(batch=batch), None)
    return model(batch)


@pytest.mark.parametrize("kind", ["ewald", "pme"])
def test_coulomb_models_cuda_match_cpu(kind):
    from nvalchemi_toolkit_b200.models.ewald import EwaldModelWrapper
    from nvalchemi_toolkit_b200.models.pme import PMEModelWrapper
    from tests.test_electrostatics import _nacl

    cls = EwaldModelWrapper if kind == "ewald" else PMEModelWrapper
    outs = {}
    for dev in ("cpu", "cuda"):
        m = cls(cutoff=5.5, accuracy=1e-8)
        m.model_config.active_outputs = {"energy", "forces", "stress", "electrostatic_potential"}
        outs[dev] = _run(m, _nacl(3, noise=0.15, seed=5, charge_noise=0.02).to(dev))
    for k in ("energy", "forces", "stress", "electrostatic_potential"):
        assert torch.allclose(outs["cuda"][k].cpu(), outs["cpu"][k], rtol=1e-9, atol=1e-9), k
    # float32 inputs: double accumulation keeps the error at single-precision input rounding
    m = cls(cutoff=5.5, accuracy=1e-6)
    m.model_config.active_outputs = {"energy", "forces"}
    b = _nacl(3, noise=0.15, seed=5).to("cuda", dtype=torch.float32)
    o = _run(m, b)
    m2 = cls(cutoff=5.5, accuracy=1e-6)
    m2.model_config.active_outputs = {"energy", "forces"}
    ref = _run(m2, _nacl(3, noise=0.15, seed=5))
    assert float((o["forces"].double().cpu() - ref["forces"]).abs().max()) < 2e-4
    assert abs(float(o["energy"]) - float(ref["energy"])) < 1e-4 * abs(float(ref["energy"]))


def test_dftd3_cuda_matches_cpu():
    from tests.test_dftd3 import _batch, _model

    cpu = _run(_model(), _batch(seed=4, n=40, box=11.0))
    gpu = _run(_model(), _batch(seed=4, n=40, box=11.0).to("cuda"))
    for k in ("energy", "forces", "virial", "coordination_numbers"):
        assert torch.allclose(gpu[k].cpu(), cpu[k], rtol=1e-9, atol=1e-11), k


def test_generic_domain_layer_on_one_gpu_matches_periodic_model():
    from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, ShardedBatch
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
    from tests.helpers import fcc_supercell

    def model():
        m = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0, switch_width=1.0)
        m.model_config.active_outputs = {"energy", "forces", "stress"}
        return m

    batch = Batch.from_data_list([fcc_supercell(4, a=5.26, z=18, noise=0.05, seed=0)]).to("cuda")
    ref = _run(model(), batch.clone())
    cfg = DomainConfig(cutoff=6.0, skin=0.0)
    sh = ShardedBatch.from_batch(batch, cfg, model().distribution_spec())
    out = DistributedModel(model(), cfg)(sh)
    assert torch.allclose(out["forces"], ref["forces"], atol=2e-5)
    assert torch.allclose(out["energy"], ref["energy"], rtol=1e-5)
    assert torch.allclose(out["stress"], ref["stress"], atol=1e-6)
