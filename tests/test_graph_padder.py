"""Fixed-shape graph padding (``distributed/graph_padder.py``)."""
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.distributed.graph_padder import (COOPadder, DenseBatchPadder, DensePadder, GraphPadder,
                                                             cap_agreement_group, resolve_cap)
from nvalchemi_toolkit_b200.models.base import NeighborListFormat
from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
from nvalchemi_toolkit_b200.neighbors import compute_neighbors
from tests.helpers import fcc_supercell


def test_resolve_cap_grows_in_buckets_and_never_shrinks():
    st = {}
    c0 = resolve_cap(st, "edges", 1000, initial_factor=1.35)
    assert c0 % 16 == 0 and c0 >= 1350
    assert resolve_cap(st, "edges", 1200, initial_factor=1.35) == c0          # inside the head-room: same bucket
    assert resolve_cap(st, "edges", 10, initial_factor=1.35) == c0            # never shrinks
    c1 = resolve_cap(st, "edges", c0 + 1, initial_factor=1.35)
    assert c1 > c0 and c1 % 16 == 0 and c1 >= int((c0 + 1) * 1.3)
    st = {}
    a0 = resolve_cap(st, "atoms", 100, initial_factor=1.0, strict_gt=False)
    assert a0 > 100                                                           # room for the dead row
    assert resolve_cap(st, "atoms", a0, strict_gt=False) > a0                 # need == cap overflows when the last row is dead
    with cap_agreement_group(None, "cpu"):                                    # single process: plain behaviour
        assert resolve_cap({}, "x", 5, initial_factor=1.0, extra=2) == 16


def test_coo_padder_keeps_energies_and_forces():
    torch.manual_seed(0)
    data = fcc_supercell(3, a=5.3, z=18, noise=0.05, dtype=torch.float64)
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0)
    b = Batch.from_data_list([data])
    compute_neighbors(b, cutoff=6.0, format=NeighborListFormat.COO)
    padder = COOPadder()
    assert isinstance(padder, GraphPadder)
    caps = {}
    p = padder.pad(b, caps)
    assert p.num_nodes == caps["atoms"] > b.num_nodes and p.num_edges == caps["edges"] > b.num_edges
    assert p.num_graphs == b.num_graphs
    nl = p.neighbor_list
    dead = caps["atoms"] - 1
    assert bool((nl[b.num_edges:] == dead).all()) and int(p.neighbor_list_shifts[b.num_edges:, 0].min()) == 1
    assert not bool((nl[: b.num_edges] >= b.num_nodes).any())
    p2 = padder.pad(b, caps)                                                  # same capacities next step
    assert (p2.num_nodes, p2.num_edges) == (p.num_nodes, p.num_edges)
    out = padder.unpad({"forces": torch.zeros(p.num_nodes, 3), "energy": torch.zeros(1, 1)}, b.num_nodes)
    assert out["forces"].shape[0] == b.num_nodes and out["energy"].shape == (1, 1)
    del model


def test_dense_batch_padder_gives_the_same_lj_result():
    data = fcc_supercell(3, a=5.3, z=18, noise=0.05, dtype=torch.float64)
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0)
    model.model_config.active_outputs = {"energy", "forces"}
    b = Batch.from_data_list([data])
    compute_neighbors(b, config=model.model_config.neighbor_config)
    ref = model(b)
    padder = DenseBatchPadder(pad_neighbors=True)
    caps = {}
    p = padder.pad(b, caps)
    assert p.num_nodes == caps["atoms"] and p.neighbor_matrix.shape == (caps["atoms"], caps["neighbors"])
    assert int(p.num_neighbors[b.num_nodes:].sum()) == 0
    out = padder.unpad(dict(model(p)), b.num_nodes)
    assert torch.allclose(out["forces"], ref["forces"], atol=1e-10)
    assert torch.allclose(out["energy"], ref["energy"], atol=1e-10)


def test_dense_padder_on_plain_dict():
    n, k = 5, 4
    data = {"positions": torch.randn(n, 3), "numbers": torch.arange(1, n + 1), "mol_idx": torch.tensor([0, 0, 1, 1, 1]),
            "neighbor_matrix": torch.tensor([[1, 2, n, n], [0, n, n, n], [3, 4, n, n], [2, n, n, n], [2, 3, n, n]]),
            "cell": torch.eye(3)}
    padder = DensePadder(row_pads={"mol_idx": DensePadder.LAST_SYSTEM})
    caps = {}
    p = padder.pad(data, caps)
    cap = caps["atoms"]
    assert p["positions"].shape == (cap, 3) and p["cell"].shape == (3, 3)
    assert p["mol_idx"][n:].tolist() == [1] * (cap - n) and int(p["numbers"][n:].sum()) == 0
    nm = p["neighbor_matrix"]
    assert nm.shape == (cap, k) and int(nm.max()) == cap - 1 and bool((nm[n:] == cap - 1).all())
    assert bool(((nm[:n] < n) | (nm[:n] == cap - 1)).all())
    out = padder.unpad({"forces": torch.ones(cap, 3), "energy": torch.ones(2)}, n)
    assert out["forces"].shape == (n, 3) and out["energy"].shape == (2,)
