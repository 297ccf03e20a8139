# SPDX-License-Identifier: Apache-2.0
"""AtomicData / Batch behaviour (mirrors the reference's test/data suite in spirit)."""
import pytest
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch
from tests.helpers import random_batch, random_molecule


def test_atomic_data_defaults_and_validation():
    d = AtomicData(atomic_numbers=torch.tensor([1, 8, 1]), positions=torch.zeros(3, 3))
    assert d.atomic_masses.shape == (3,) and abs(float(d.atomic_masses[1]) - 15.999) < 1e-3
    assert d.velocities.shape == (3, 3) and d.atom_categories.dtype == torch.long
    with pytest.raises(ValueError):
        AtomicData(atomic_numbers=torch.tensor([1, 8]), positions=torch.zeros(3, 3))
    with pytest.raises(ValueError):
        AtomicData(atomic_numbers=torch.tensor([1, 8]), positions=torch.zeros(2, 3), forces=torch.zeros(3, 3))


def test_atomic_data_dtype_cast_warns():
    with pytest.warns(UserWarning):
        d = AtomicData(atomic_numbers=torch.tensor([1]), positions=torch.zeros(1, 3), forces=torch.zeros(1, 3, dtype=torch.float64))
    assert d.forces.dtype == torch.float32


def test_chemical_hash_is_order_invariant():
    a = random_molecule(6, 1)
    perm = torch.randperm(6)
    b = AtomicData(atomic_numbers=a.atomic_numbers[perm], positions=a.positions[perm])
    assert a.chemical_hash == b.chemical_hash
    c = AtomicData(atomic_numbers=a.atomic_numbers, positions=a.positions + 0.1)
    assert a.chemical_hash != c.chemical_hash


def test_batch_roundtrip_and_offsets(device):
    sizes = [3, 5, 2]
    data = [random_molecule(n, i, n_edges=4, periodic=True) for i, n in enumerate(sizes)]
    b = Batch.from_data_list(data, device=device)
    assert b.num_graphs == 3 and b.num_nodes == 10 and b.num_edges == 12
    assert b.batch_ptr.tolist() == [0, 3, 8, 10] and b.batch_idx.dtype == torch.int32
    assert b.cell.shape == (3, 3, 3) and b.energy.shape == (3, 1)
    for i, d in enumerate(data):
        got = b.get_data(i)
        assert torch.equal(got.neighbor_list.cpu(), d.neighbor_list)
        assert torch.allclose(got.positions.cpu(), d.positions)
    sel = b.index_select([2, 0])
    assert sel.num_nodes == 5
    assert torch.equal(sel.neighbor_list[:4].cpu(), data[2].neighbor_list)
    assert torch.equal(sel.neighbor_list[4:].cpu(), data[0].neighbor_list + 2)


def test_put_defrag_trim(device):
    b = random_batch([3, 5, 2], n_edges=3, periodic=True, device=device)
    ref = [b.get_data(i) for i in range(3)]
    buf = Batch.empty(num_systems=4, num_nodes=8, num_edges=12, template=b, device=device)
    assert buf.num_graphs == 0
    buf.put(b, torch.tensor([True, True, True], device=device))
    assert b._copied_mask.tolist() == [True, True, False]  # third does not fit in 8 atoms
    assert buf.num_graphs == 2 and buf.num_nodes == 8
    assert torch.equal(buf.get_data(1).neighbor_list.cpu(), ref[1].neighbor_list.cpu())
    b.defrag()
    assert b.num_graphs == 1 and torch.equal(b.neighbor_list.cpu(), ref[2].neighbor_list.cpu())
    buf.defrag(torch.tensor([True, False], device=device))
    assert buf.num_graphs == 1 and buf.system_capacity == 4
    assert torch.allclose(buf.positions.cpu(), ref[1].positions.cpu())
    assert torch.equal(buf.neighbor_list.cpu(), ref[1].neighbor_list.cpu())
    t = buf.trim(torch.tensor([True], device=device))
    assert t is None


def test_append_add_key_and_moves():
    b = random_batch([3, 4], n_edges=2)
    other = random_batch([5], seed=9, n_edges=2)
    b.append(other)
    assert b.num_graphs == 3 and b.num_nodes == 12 and int(b.neighbor_list[-2:].min()) >= 7
    b.add_key("status", torch.zeros(3, 1, dtype=torch.long), level="system")
    assert b.status.shape == (3, 1)
    with pytest.raises(KeyError):
        b.add_key("status", torch.zeros(3, 1, dtype=torch.long), level="system")
    c = b.clone().to(dtype=torch.float64)
    assert c.positions.dtype == torch.float64 and c.atomic_numbers.dtype == torch.long
    assert "positions" in b and len(b) == 3
    assert b[1].num_nodes == 4 and b[[0, 2]].num_graphs == 2


def test_from_raw_dicts_skips_validation():
    dicts = [{"positions": torch.zeros(2, 3), "atomic_numbers": torch.tensor([1, 1]), "energy": torch.zeros(1, 1),
              "my_field": torch.ones(2, 4)} for _ in range(3)]
    b = Batch.from_raw_dicts(dicts, field_levels={"my_field": "node"})
    assert b.my_field.shape == (6, 4) and b.num_graphs == 3


def test_reference_package_name_alias():
    from nvalchemi_toolkit_b200 import compat

    compat.install_alias()
    try:
        import nvalchemi  # noqa: F401
        from nvalchemi.data import AtomicData as A
        from nvalchemi.dynamics import NVE as N
        from nvalchemi.models.lj import LennardJonesModelWrapper as L

        import nvalchemi_toolkit_b200 as real
        from nvalchemi_toolkit_b200.dynamics import NVE
        from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper

        assert nvalchemi is real and A is real.AtomicData and N is NVE and L is LennardJonesModelWrapper
    finally:
        compat.remove_alias()


def _fill_and_drain(device, planned: bool, monkeypatch):
    """Three puts into a fixed buffer interleaved with a defrag; returns the observable state after every stage."""
    import nvalchemi_toolkit_b200.data.batch as batch_mod

    if not planned:
        monkeypatch.setattr(batch_mod, "_buffer_ops", lambda: None)
    src1 = random_batch([3, 5, 2, 4], n_edges=3, periodic=True, device=device, seed=1)
    src2 = random_batch([2, 6, 1], n_edges=2, periodic=True, device=device, seed=2)
    buf = Batch.empty(num_systems=5, num_nodes=14, num_edges=14, template=src1, device=device)
    out = []

    def snap(tag):
        out.append((tag, buf.num_graphs, buf.num_nodes, buf.num_edges, buf.batch_ptr.cpu().clone(), buf.positions.cpu().clone(),
                    buf.neighbor_list.cpu().clone(), buf.cell.cpu().clone()))

    buf.put(src1, torch.tensor([True, False, True, True], device=device))  # 3 + 2 + 4 atoms, 9 edges
    c1 = src1._copied_mask.cpu().clone()
    buf.put(src2, torch.tensor([True, True, True], device=device))          # chained: counts not read in between
    c2 = src2._copied_mask.cpu().clone()
    snap("after puts")
    buf.defrag(torch.tensor([False, True, False, True, False], device=device)[: buf.num_graphs])
    snap("after defrag")
    buf.put(src1, torch.tensor([False, True, False, False], device=device))
    snap("after refill")
    return out, c1, c2


def test_planned_put_defrag_matches_index_path(device, monkeypatch):
    """``Batch.put`` / ``defrag`` through the device planners leave the same buffer as the index-list fallback."""
    from nvalchemi_toolkit_b200.data.level_storage import _buffer_ops

    if _buffer_ops() is None:
        pytest.skip("native library not built")
    got, g1, g2 = _fill_and_drain(device, True, monkeypatch)
    want, w1, w2 = _fill_and_drain(device, False, monkeypatch)
    assert torch.equal(g1, w1) and torch.equal(g2, w2)
    for a, b in zip(got, want):
        assert a[:4] == b[:4], (a[:4], b[:4])
        for x, y in zip(a[4:], b[4:]):
            assert torch.equal(x, y), a[0]


@pytest.mark.gpu
def test_planned_put_makes_no_host_sync():
    """On the GPU a masked put followed by a second one runs without a single host synchronisation; the counts are read
    back once, when the host asks for them."""
    src = random_batch([3, 5, 2, 4], n_edges=3, periodic=True, device="cuda", seed=1)
    buf = Batch.empty(num_systems=8, num_nodes=64, num_edges=64, template=src, device="cuda")
    m = torch.tensor([True, False, True, True], device="cuda")
    src.batch_ptr, src.edge_ptr, src._edges_group.batch_idx  # derived CSR views of the source exist before the region
    buf.put(src, m)  # first call builds the buffer's device-side CSR
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        buf.put(src, m)
        buf.put(src, m)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    assert buf.num_graphs == 8 and buf.num_nodes == 9 * 2 + 3 + 2


def test_lazy_counts_after_planned_put(device):
    """After a planned put the host counts are pending (still on the device) until first read; the derived CSR views and a
    host-path modification afterwards see the resolved values."""
    from nvalchemi_toolkit_b200.data.level_storage import _buffer_ops

    if _buffer_ops() is None:
        pytest.skip("native library not built")
    src = random_batch([3, 5, 2], n_edges=2, periodic=True, device=device, seed=4)
    buf = Batch.empty(num_systems=6, num_nodes=32, num_edges=32, template=src, device=device)
    buf.put(src, torch.tensor([True, False, True], device=device))
    atoms = buf._atoms_group
    assert atoms._pending is not None and buf._system_group._pending is not None
    ptr, count = atoms.device_csr()
    assert int(count) == 2 and ptr[:3].tolist() == [0, 3, 5]
    assert buf.num_graphs == 2 and atoms._pending is None            # resolved by the read
    assert buf.num_nodes == 5 and buf.num_edges == 4
    assert buf.batch_ptr.tolist() == [0, 3, 5] and buf.batch_idx.tolist() == [0, 0, 0, 1, 1]
    assert atoms.lengths[:3].tolist() == [3, 2, 0]
    buf.put(src, torch.tensor([False, True, False], device=device))   # counts pending again, then a host-path append
    more = random_batch([4], n_edges=2, periodic=True, device=device, seed=9)
    buf.put(more, torch.tensor([True], device=device))
    assert buf.num_graphs == 4 and buf.num_nodes == 14 and buf.batch_ptr.tolist() == [0, 3, 5, 10, 14]
    got = buf.get_data(2)
    assert torch.equal(got.positions.cpu(), src.get_data(1).positions.cpu())
    assert torch.equal(got.neighbor_list.cpu(), src.get_data(1).neighbor_list.cpu())
