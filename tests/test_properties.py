# SPDX-License-Identifier: Apache-2.0
"""Property-based tests (hypothesis): invariants that must hold for ANY input of the stated shape, checked against
brute-force or list-based restatements written here."""
import itertools
import math

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200 import neighbors as nb
from tests.helpers import random_batch, random_molecule

SETTINGS = dict(max_examples=25, deadline=None)


# ---------------------------------------------------------------------------------------------------- neighbour lists
def _brute_force(pos, cell, pbc, cutoff):
    """{(i, j, sx, sy, sz)} with |r_j + S.cell - r_i| < cutoff, enumerating enough periodic images explicitly."""
    inv = torch.linalg.inv(cell)
    heights = 1.0 / inv.norm(dim=0)                      # distance between opposite faces, per lattice direction
    reach = [int(math.ceil(cutoff / float(h))) if p else 0 for h, p in zip(heights, pbc)]
    out = set()
    n = pos.shape[0]
    for s in itertools.product(*[range(-r, r + 1) for r in reach]):
        shift = torch.tensor(s, dtype=pos.dtype) @ cell
        d = (pos[None, :, :] + shift - pos[:, None, :]).norm(dim=-1)
        hit = d < cutoff
        if s == (0, 0, 0):
            hit &= ~torch.eye(n, dtype=torch.bool)
        for i, j in hit.nonzero().tolist():
            out.add((i, j) + s)
    return out


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), n=st.integers(2, 24), pbc=st.tuples(st.booleans(), st.booleans(), st.booleans()),
       skew=st.floats(0.0, 0.45), cutoff=st.floats(1.5, 4.5))
def test_neighbor_matrix_equals_brute_force_on_random_triclinic_cells(seed, n, pbc, skew, cutoff):
    g = torch.Generator().manual_seed(seed)
    cell = torch.diag(4.0 + 3.0 * torch.rand(3, generator=g, dtype=torch.float64))
    cell[1, 0], cell[2, 0], cell[2, 1] = skew * cell[0, 0], -skew * cell[0, 0], skew * cell[1, 1]
    pos = torch.rand(n, 3, generator=g, dtype=torch.float64) @ cell
    pbc_t = torch.tensor(pbc)
    bidx, bptr = torch.zeros(n, dtype=torch.int32), torch.tensor([0, n], dtype=torch.int32)
    nm, num, sh = nb.neighbor_matrix(pos, cell[None], pbc_t[None], bidx, bptr, cutoff, 512)
    got = set()
    for i in range(n):
        for k in range(int(num[i])):
            got.add((i, int(nm[i, k])) + tuple(int(x) for x in sh[i, k]))
    want = _brute_force(pos, cell, pbc, cutoff)
    # pairs within 1e-9 of the cutoff may fall on either side
    def near(entry):
        i, j, *s = entry
        d = (pos[j] + torch.tensor(s, dtype=pos.dtype) @ cell - pos[i]).norm()
        return abs(float(d) - cutoff) < 1e-9
    assert {e for e in got ^ want if not near(e)} == set()
    assert int(num.sum()) == len(got)  # no duplicate (j, shift) entries in a row


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 9), min_size=1, max_size=5))
def test_neighbor_lists_never_cross_systems_of_a_batch(seed, sizes):
    b = random_batch(sizes, seed=seed, periodic=True)
    nb.compute_neighbors(b, 4.0)
    owner = b.batch_idx.long()
    n = b.num_nodes
    for i in range(n):
        for k in range(int(b.num_neighbors[i])):
            assert owner[int(b.neighbor_matrix[i, k])] == owner[i]
    assert bool((b.neighbor_matrix[torch.arange(b.neighbor_matrix.shape[1])[None, :] >= b.num_neighbors[:, None]] == n).all())


# ---------------------------------------------------------------------------------------------------- batches
@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 7), min_size=1, max_size=6), edges=st.integers(0, 5))
def test_batch_round_trip_and_selection(seed, sizes, edges):
    data = [random_molecule(n, seed + i, n_edges=edges) for i, n in enumerate(sizes)]
    b = Batch.from_data_list(data)
    assert b.num_graphs == len(sizes) and b.num_nodes == sum(sizes)
    assert b.batch_ptr.tolist() == [0] + list(itertools.accumulate(sizes))
    back = b.to_data_list()
    for d, e in zip(data, back):
        assert torch.equal(d.positions, e.positions) and torch.equal(d.atomic_numbers, e.atomic_numbers)
        if edges:
            assert torch.equal(d.neighbor_list, e.neighbor_list)       # edge indices come back system-local
    g = torch.Generator().manual_seed(seed)
    pick = torch.randperm(len(sizes), generator=g)[: max(1, len(sizes) // 2)].tolist()
    sub = b.index_select(pick)
    assert sub.num_graphs == len(pick) and sub.num_nodes == sum(sizes[i] for i in pick)
    for k, i in enumerate(pick):
        assert torch.equal(sub[k].positions, data[i].positions)
    both = Batch.from_data_list(data)
    both.append(sub)
    assert both.num_graphs == len(sizes) + len(pick) and torch.equal(both[len(sizes)].positions, data[pick[0]].positions)


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 6), min_size=2, max_size=6),
       incoming=st.lists(st.integers(1, 6), min_size=1, max_size=5))
def test_put_and_defrag_keep_exactly_the_systems_a_list_would(seed, sizes, incoming):
    """Graduate a random subset, compact, then refill from a source batch: the live systems equal what plain Python list
    operations on the per-system data give, in order."""
    g = torch.Generator().manual_seed(seed)
    data = [random_molecule(n, seed + i) for i, n in enumerate(sizes)]
    src_data = [random_molecule(n, seed + 100 + i) for i, n in enumerate(incoming)]
    cap_atoms = sum(sizes) + sum(incoming)
    buf = Batch.empty(num_systems=len(sizes) + len(incoming), num_nodes=cap_atoms, num_edges=0, template=Batch.from_data_list(data))
    buf.put(Batch.from_data_list(data), torch.ones(len(sizes), dtype=torch.bool))
    gone = torch.rand(len(sizes), generator=g) < 0.5
    buf.defrag(gone)
    expect = [d for d, x in zip(data, gone.tolist()) if not x]
    take = torch.rand(len(incoming), generator=g) < 0.7
    buf.put(Batch.from_data_list(src_data), take)
    expect += [d for d, x in zip(src_data, take.tolist()) if x]
    assert buf.num_graphs == len(expect)
    for k, d in enumerate(expect):
        assert torch.equal(buf[k].positions, d.positions) and torch.equal(buf[k].atomic_numbers, d.atomic_numbers)


# ---------------------------------------------------------------------------------------------------- storage
@settings(max_examples=20, deadline=None)
@given(seed=st.integers(0, 10_000), rows=st.integers(1, 200), width=st.integers(1, 5), chunk=st.integers(1, 64),
       shards=st.sampled_from([None, 1, 2, 4]), compressor=st.sampled_from([None, "gzip", "zstd"]),
       dtype=st.sampled_from(["float32", "float64", "int64", "uint8"]))
def test_zarr_array_round_trips_any_chunking(tmp_path_factory, seed, rows, width, chunk, shards, compressor, dtype):
    """Appends of uneven sizes, a partial overwrite and range reads return exactly what was written, whatever the chunk
    size, shard size, codec and element type."""
    import numpy as np

    from nvalchemi_toolkit_b200.data.zarr_store import ZarrArray, ZarrArrayConfig

    rng = np.random.default_rng(seed)
    full = (rng.standard_normal((rows, width)) * 100).astype(dtype)
    cfg = ZarrArrayConfig(chunk_rows=chunk, compressor=compressor, shard_rows=None if shards is None else shards * chunk)
    arr = ZarrArray.create(tmp_path_factory.mktemp("z") / "a", (0, width), dtype, cfg)
    pos = 0
    while pos < rows:
        step = int(rng.integers(1, max(2, rows // 3 + 1)))
        arr.append(full[pos: pos + step])
        pos += step
    assert arr.shape == (rows, width)
    lo = int(rng.integers(0, rows))
    hi = int(rng.integers(lo, rows)) + 1
    patch = (rng.standard_normal((hi - lo, width)) * 7).astype(dtype)
    arr.write(lo, patch)
    full[lo:hi] = patch
    again = ZarrArray(arr.path)  # a fresh handle reads the files, not a cache
    assert np.array_equal(again.read(), full)
    a, b = sorted(int(x) for x in rng.integers(0, rows + 1, size=2))
    assert np.array_equal(again.read(a, b), full[a:b])


# ---------------------------------------------------------------------------------------------------- sampling / losses
@settings(**SETTINGS)
@given(weights=st.lists(st.floats(0.0, 50.0), min_size=1, max_size=8), total=st.integers(0, 500))
def test_counts_from_weights_are_exact_and_within_one_of_proportional(weights, total):
    from nvalchemi_toolkit_b200.data.datapipes import counts_from_weights

    if sum(weights) <= 0:
        with pytest.raises(ValueError):
            counts_from_weights(weights, total)
        return
    counts = counts_from_weights(weights, total)
    assert sum(counts) == total and all(c >= 0 for c in counts)
    for c, w in zip(counts, weights):
        assert abs(c - total * w / sum(weights)) < 1.0 + 1e-9
        assert w > 0 or c == 0


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 6), min_size=1, max_size=6), frac=st.floats(0.0, 1.0))
def test_masked_losses_equal_losses_on_the_labelled_subset(seed, sizes, frac):
    """``ignore_nonfinite``: the value equals the plain loss evaluated on the labelled graphs only, and predictions of
    unlabelled graphs receive exactly zero gradient."""
    from nvalchemi_toolkit_b200.training.losses import EnergyMSELoss, ForceMSELoss

    g = torch.Generator().manual_seed(seed)
    b = random_batch(sizes, seed=seed)
    nG, n = len(sizes), sum(sizes)
    b.energy = torch.randn(nG, 1, generator=g)
    b.forces = torch.randn(n, 3, generator=g)
    missing = torch.rand(nG, generator=g) < frac
    pe = torch.randn(nG, 1, generator=g, requires_grad=True)
    pf = torch.randn(n, 3, generator=g, requires_grad=True)
    labelled = (~missing).nonzero().reshape(-1).tolist()
    energy, forces = b.energy.clone(), b.forces.clone()
    b.energy = torch.where(missing[:, None], torch.full_like(energy, float("nan")), energy)
    atom_missing = missing[b.batch_idx.long()]
    b.forces = torch.where(atom_missing[:, None], torch.full_like(forces, float("inf")), forces)
    le = EnergyMSELoss(ignore_nonfinite=True)({"energy": pe}, b)
    lf = ForceMSELoss(ignore_nonfinite=True)({"forces": pf}, b)
    (le + lf).backward()
    assert torch.isfinite(pe.grad).all() and torch.isfinite(pf.grad).all()
    assert float(pe.grad[missing].abs().sum()) == 0.0 and float(pf.grad[atom_missing].abs().sum()) == 0.0
    if not labelled:
        assert float(le.detach()) == 0.0 and float(lf.detach()) == 0.0
        return
    sub = b.index_select(labelled)
    sub.energy, sub.forces = energy[labelled], forces[~atom_missing]
    want_e = EnergyMSELoss()({"energy": pe.detach()[labelled]}, sub)
    want_f = ForceMSELoss()({"forces": pf.detach()[~atom_missing]}, sub)
    assert float(le.detach()) == pytest.approx(float(want_e), rel=1e-5, abs=1e-7)
    assert float(lf.detach()) == pytest.approx(float(want_f), rel=1e-5, abs=1e-7)


# ---------------------------------------------------------------------------------------------------- decomposition
@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), world=st.sampled_from([1, 2, 3, 4, 6, 8, 12]), n=st.integers(1, 200),
       pbc=st.tuples(st.booleans(), st.booleans(), st.booleans()), skew=st.floats(0.0, 0.4))
def test_spatial_partition_owns_every_atom_once_and_neighbours_are_mutual(seed, world, n, pbc, skew):
    from nvalchemi_toolkit_b200.distributed.partitioner import SpatialPartitioner

    g = torch.Generator().manual_seed(seed)
    cell = torch.diag(20.0 + 20.0 * torch.rand(3, generator=g, dtype=torch.float64))
    cell[1, 0], cell[2, 1] = skew * cell[0, 0], -skew * cell[1, 1]
    part = SpatialPartitioner(cell, torch.tensor(pbc), world, cutoff=4.0)
    assert part.grid[0] * part.grid[1] * part.grid[2] == world
    # atoms anywhere in space (also outside the cell): wrapped or clamped into exactly one box
    pos = (torch.rand(n, 3, generator=g, dtype=torch.float64) * 3.0 - 1.0) @ cell
    owner = part.assign_atoms_to_ranks(pos)
    assert owner.shape == (n,) and int(owner.min()) >= 0 and int(owner.max()) < world
    assert bool(part.keeps_owner(pos, owner)[(part.fractional(pos) >= 0).all(-1) & (part.fractional(pos) < 1).all(-1)].all())
    frac = part.fractional(pos)
    inside = ((frac >= 0) & (frac < 1)).all(-1)
    for r in range(world):
        lo, hi = part.box(r)
        mine = inside & (owner == r)
        assert bool(((frac[mine] >= lo - 1e-12) & (frac[mine] <= hi + 1e-12)).all())
        for other in part.neighbor_ranks(r):
            assert other != r and r in part.neighbor_ranks(other)


# ---------------------------------------------------------------------------------------------------- level storages
@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), ops=st.lists(st.sampled_from(["put", "defrag"]), min_size=1, max_size=8))
def test_level_storages_follow_a_list_model_through_random_put_and_defrag(seed, ops):
    """A fixed-capacity segmented storage (atoms of several systems) and a uniform one (one row per system) driven by
    the same random sequence of appends and compactions always hold exactly what a Python list of segments holds."""
    from nvalchemi_toolkit_b200.data.level_storage import SegmentedLevelStorage, UniformLevelStorage

    g = torch.Generator().manual_seed(seed)
    seg_cap, elem_cap = 12, 60
    seg = SegmentedLevelStorage({"x": torch.zeros(elem_cap, 2), "z": torch.zeros(elem_cap, dtype=torch.int64)},
                                torch.zeros(seg_cap, dtype=torch.int32), num_segments=0, num_elements=0,
                                segment_capacity=seg_cap, element_capacity=elem_cap)
    uni = UniformLevelStorage({"e": torch.zeros(seg_cap, 1)}, num_valid=0, capacity=seg_cap)
    model: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = []   # (x rows, z rows, e row) per live segment
    for op in ops:
        if op == "put":
            k = int(torch.randint(1, 4, (1,), generator=g))
            lens = torch.randint(1, 6, (k,), generator=g)
            xs = [torch.randn(int(n), 2, generator=g) for n in lens]
            zs = [torch.randint(1, 90, (int(n),), generator=g) for n in lens]
            es = torch.randn(k, 1, generator=g)
            src = SegmentedLevelStorage({"x": torch.cat(xs), "z": torch.cat(zs)}, lens.to(torch.int32))
            src_u = UniformLevelStorage({"e": es})
            take = torch.nonzero(torch.rand(k, generator=g) < 0.7).flatten()
            # what fits, in order (the storages raise when asked for more than they can hold)
            fit = []
            n_seg, n_el = len(model), sum(m[0].shape[0] for m in model)
            for t in take.tolist():
                if n_seg + 1 <= seg_cap and n_el + int(lens[t]) <= elem_cap:
                    fit.append(t)
                    n_seg, n_el = n_seg + 1, n_el + int(lens[t])
            fit_t = torch.tensor(fit, dtype=torch.int64)
            seg.put(src, fit_t)
            uni.put(src_u, fit_t)
            model += [(xs[t], zs[t], es[t]) for t in fit]
            if take.numel() > len(fit) and take.numel() > 0:
                with pytest.raises(ValueError):
                    huge = SegmentedLevelStorage({"x": torch.zeros(elem_cap + 1, 2), "z": torch.zeros(elem_cap + 1, dtype=torch.int64)},
                                                 torch.tensor([elem_cap + 1], dtype=torch.int32))
                    seg.put(huge, torch.tensor([0]))
        else:
            if not model:
                continue
            keep = torch.nonzero(torch.rand(len(model), generator=g) < 0.6).flatten()
            seg.defrag(keep)
            uni.defrag(keep)
            model = [model[i] for i in keep.tolist()]
        assert seg.num_segments == uni.num_valid == len(model)
        assert seg.num_elements == sum(m[0].shape[0] for m in model)
        assert seg.batch_ptr.tolist() == [0] + list(itertools.accumulate(m[0].shape[0] for m in model))
        if model:
            assert torch.equal(seg["x"], torch.cat([m[0] for m in model])) and torch.equal(seg["z"], torch.cat([m[1] for m in model]))
            assert torch.equal(uni["e"], torch.stack([m[2] for m in model]))
            assert seg.batch_idx.tolist() == [i for i, m in enumerate(model) for _ in range(m[0].shape[0])]
        assert seg.free_segments() == seg_cap - len(model) and uni.free_rows() == seg_cap - len(model)


# ---------------------------------------------------------------------------------------------------- integrators
@settings(max_examples=8, deadline=None)
@given(seed=st.integers(0, 1000), n_cells=st.sampled_from([2, 3]), dt=st.floats(0.5, 2.0), steps=st.integers(3, 12))
def test_velocity_verlet_is_time_reversible_and_conserves_momentum(seed, n_cells, dt, steps):
    """NVE with a conservative pair potential: total momentum stays put, and after flipping the velocities the same
    number of steps retraces the trajectory to the starting point (float64, tolerances of rounding only)."""
    from nvalchemi_toolkit_b200.dynamics import NVE, _ops
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
    from tests.helpers import fcc_supercell

    batch = Batch.from_data_list([fcc_supercell(n_cells, a=5.26, z=18, noise=0.05, seed=seed, dtype=torch.float64)])
    model = LennardJonesModelWrapper(epsilon=0.0104, sigma=3.4, cutoff=6.0, switch_width=1.0)
    model.model_config.active_outputs = {"energy", "forces"}
    _ops.initialize_velocities(batch.velocities, batch.atomic_masses, 120.0, batch.batch_idx, random_seed=seed)
    x0, v0 = batch.positions.clone(), batch.velocities.clone()
    p0 = (batch.atomic_masses[:, None] * v0).sum(0)
    dyn = NVE(model, dt=dt, hooks=model.make_neighbor_hooks())
    from nvalchemi_toolkit_b200.dynamics import DynamicsStage

    dyn._call_hooks(DynamicsStage.BEFORE_COMPUTE, batch)   # the batch carries placeholder forces (zeros): evaluate the
    dyn.compute(batch)                                      # real ones before the first half kick
    dyn.run(batch, steps)
    p1 = (batch.atomic_masses[:, None] * batch.velocities).sum(0)
    assert torch.allclose(p1, p0, atol=1e-9)
    assert float((batch.positions - x0).abs().max()) > 1e-4          # it did move
    batch.velocities.mul_(-1.0)
    dyn.run(batch, steps)
    assert torch.allclose(batch.positions, x0, atol=1e-9) and torch.allclose(-batch.velocities, v0, atol=1e-9)


# ---------------------------------------------------------------------------------------------------- inflight sampler
@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 12), min_size=1, max_size=14), max_atoms=st.integers(12, 40),
       max_batch=st.one_of(st.none(), st.integers(1, 6)), bin_width=st.integers(1, 5), shuffle=st.booleans())
def test_size_aware_sampler_respects_budgets_and_hands_out_each_sample_once(seed, sizes, max_atoms, max_batch, bin_width, shuffle):
    from nvalchemi_toolkit_b200.data.datapipes import InMemoryDataset
    from nvalchemi_toolkit_b200.dynamics.sampler import SizeAwareSampler

    import random as _random

    _random.seed(seed)
    data = [random_molecule(n, seed + i) for i, n in enumerate(sizes)]
    sampler = SizeAwareSampler(InMemoryDataset(data), max_atoms=max_atoms, max_batch_size=max_batch, bin_width=bin_width,
                               shuffle=shuffle)
    first = sampler.build_initial_batch()
    assert first.num_nodes <= max_atoms and (max_batch is None or first.num_graphs <= max_batch)
    seen_ids = first.system_id.reshape(-1).tolist() if getattr(first, "system_id", None) is not None else []
    handed = sorted(first.num_nodes_per_graph.tolist())
    # free a random slot budget repeatedly until the supply is exhausted
    g = torch.Generator().manual_seed(seed)
    for _ in range(4 * len(sizes)):
        if sampler.exhausted:
            break
        budget = int(torch.randint(1, max_atoms + 1, (1,), generator=g))
        got = sampler.request_replacements_budget(atom_budget=budget, max_count=3)
        assert sum(d.num_nodes for d in got) <= budget and len(got) <= 3
        handed += [d.num_nodes for d in got]
        seen_ids += [int(d.system_id) for d in got if getattr(d, "system_id", None) is not None]
        one = sampler.request_replacement(budget, 10 ** 9)
        if one is not None:
            assert one.num_nodes <= budget
            handed.append(one.num_nodes)
            if getattr(one, "system_id", None) is not None:
                seen_ids.append(int(one.system_id))
    assert len(seen_ids) == len(set(seen_ids))                      # ids are unique over the whole run
    remaining = len(sampler)
    assert len(handed) + remaining == len(sizes)                    # nothing handed out twice, nothing lost
    if sampler.exhausted:
        assert sorted(handed) == sorted(sizes)
        assert sampler.request_replacement(max_atoms, 10 ** 9) is None


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), lengths=st.lists(st.integers(1, 9), min_size=1, max_size=4), world=st.integers(1, 4),
       replacement=st.booleans(), shuffle=st.booleans(), drop_last=st.booleans(), extra=st.integers(0, 7))
def test_multidataset_sampler_shards_one_epoch_order_evenly(seed, lengths, world, replacement, shuffle, drop_last, extra):
    from nvalchemi_toolkit_b200.data.datapipes import InMemoryDataset, MultiDataset, MultiDatasetSampler, counts_from_weights

    multi = MultiDataset([InMemoryDataset([random_molecule(2, seed + 10 * k + i) for i in range(n)]) for k, n in enumerate(lengths)])
    num_samples = len(multi) + extra
    ranks = [MultiDatasetSampler(multi, num_samples=num_samples, seed=seed, rank=r, world_size=world, replacement=replacement,
                                 shuffle=shuffle, drop_last=drop_last) for r in range(world)]
    shares = [list(s) for s in ranks]
    per = num_samples // world if drop_last else -(-num_samples // world)
    assert all(len(sh) == per == len(s) for sh, s in zip(shares, ranks))          # every rank runs the same number of steps
    order = ranks[0].epoch_order()
    assert all(r.epoch_order() == order for r in ranks)                            # one order, known to all ranks
    merged = [shares[i % world][i // world] for i in range(per * world)]           # undo the strided split
    head = order[: per * world] if drop_last else order + order[: per * world - len(order)]
    assert merged == head
    # exact per-dataset counts in the epoch, proportional to the dataset lengths
    want = counts_from_weights([float(n) for n in lengths], num_samples)
    got = [sum(1 for i in order if multi.locate(i)[0] == k) for k in range(len(lengths))]
    assert got == want
    if not replacement:
        for k, n in enumerate(lengths):                                            # no repeats before a dataset is exhausted
            mine = [i for i in order if multi.locate(i)[0] == k]
            assert len(set(mine)) == min(len(mine), n)
    for s in ranks:
        s.set_epoch(1)
    assert ranks[0].epoch_order() == ranks[-1].epoch_order()


# ---------------------------------------------------------------------------------------------------- halo exchange
@settings(max_examples=15, deadline=None)
@given(seed=st.integers(0, 10_000), n_cells=st.sampled_from([2, 3]), cutoff=st.floats(2.5, 6.0), width=st.integers(1, 4),
       pbc=st.tuples(st.booleans(), st.booleans(), st.booleans()))
def test_halo_forward_and_reverse_are_adjoint_and_ghosts_are_images(seed, n_cells, cutoff, width, pbc):
    """One rank, periodic images as ghosts: the reverse exchange is the transpose of the forward one
    (<forward(x), y> = <x, reverse(y)>, which is what makes forces on ghost copies return correctly), and every ghost
    position is its owner's position displaced by a lattice vector."""
    from nvalchemi_toolkit_b200.distributed import DomainConfig, ShardedBatch
    from nvalchemi_toolkit_b200.distributed.spec import SPEC_LJ_HALO
    from tests.helpers import fcc_supercell

    d = fcc_supercell(n_cells, a=4.0, z=29, noise=0.1, seed=seed, dtype=torch.float64)
    d.pbc = torch.tensor(pbc)
    batch = Batch.from_data_list([d])
    sh = ShardedBatch.from_batch(batch, DomainConfig(cutoff=cutoff, skin=0.0), SPEC_LJ_HALO)
    halo, n, ng = sh.halo, sh.n_owned, sh.n_ghost
    assert n == batch.num_nodes
    if not any(pbc):
        assert ng == 0
        return
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, width, generator=g, dtype=torch.float64)
    y = torch.randn(ng, width, generator=g, dtype=torch.float64)
    lhs = (halo.forward(x) * y).sum()
    rhs = (x * halo.reverse_add(y, torch.zeros_like(x))).sum()
    assert float(lhs) == pytest.approx(float(rhs), rel=1e-10, abs=1e-10)
    padded = sh.padded_batch(halo)
    owner_row = halo.forward(torch.arange(n, dtype=torch.float64).reshape(-1, 1)).reshape(-1).long()
    disp = padded.positions[n:] - padded.positions[:n][owner_row]   # owned rows may have been wrapped into the cell
    frac = disp @ torch.linalg.inv(batch.cell.reshape(3, 3))
    assert torch.allclose(frac, frac.round(), atol=1e-9) and bool((frac.round().abs().sum(-1) > 0).all())
    assert bool((frac.round()[:, ~torch.tensor(pbc)] == 0).all())     # no images along open directions
    # every ghost lies within the ghost width of the cell (it could be somebody's neighbour), none deep inside
    inside = (padded.positions[n:] @ torch.linalg.inv(batch.cell.reshape(3, 3)))
    assert bool(((inside < 0) | (inside > 1)).any(-1).all())


# ---------------------------------------------------------------------------------------------------- data loader
@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), n=st.integers(1, 23), batch_size=st.integers(1, 6), world=st.integers(1, 4),
       shuffle=st.booleans(), drop_last=st.booleans(), epoch=st.integers(0, 3))
def test_dataloader_epochs_resume_points_and_rank_shares(seed, n, batch_size, world, shuffle, drop_last, epoch):
    """Every rank sees the same number of batches; together the ranks cover every sample; a loader told to resume at
    batch k yields exactly the tail of the epoch; the order depends on (seed, epoch) only."""
    from nvalchemi_toolkit_b200.data.datapipes import DataLoader, InMemoryDataset

    data = [random_molecule(1 + i % 3, seed + i) for i in range(n)]
    for i, d in enumerate(data):
        d.add_system_property("tag", torch.tensor([[float(i)]]))

    def tags(loader):
        return [[int(t) for t in b.tag.reshape(-1).tolist()] for b in loader]

    loaders = []
    for r in range(world):
        dl = DataLoader(InMemoryDataset(data), batch_size=batch_size, shuffle=shuffle, drop_last=drop_last, seed=seed)
        dl.set_distributed(r, world)
        dl.set_epoch(epoch)
        loaders.append(dl)
    per_rank = [tags(dl) for dl in loaders]
    assert len({len(x) for x in per_rank}) == 1 and all(len(dl) == len(per_rank[0]) for dl in loaders)
    seen = {t for x in per_rank for b in x for t in b}
    if not drop_last:
        assert seen == set(range(n))
    assert all(len(b) == batch_size for x in per_rank for b in x[:-1])
    again = tags(loaders[0])
    assert again == per_rank[0]                                   # same (seed, epoch): same order
    if shuffle and n > 4 and world == 1:
        loaders[0].set_epoch(epoch + 1)
        assert tags(loaders[0]) != per_rank[0] or n <= batch_size
        loaders[0].set_epoch(epoch)
    k = len(per_rank[0]) // 2
    loaders[0].set_epoch_step(k)
    assert tags(loaders[0]) == per_rank[0][k:]
    assert tags(loaders[0]) == per_rank[0]                        # the resume point applies to one iteration only


@settings(max_examples=15, deadline=None)
@given(seed=st.integers(0, 10_000), sizes=st.lists(st.integers(1, 7), min_size=1, max_size=6), edges=st.integers(0, 4),
       chunk=st.integers(1, 16), compressor=st.sampled_from([None, "gzip"]))
def test_zarr_dataset_round_trips_samples_with_custom_fields_of_every_level(tmp_path_factory, seed, sizes, edges, chunk, compressor):
    """Write structures with a custom per-atom, per-edge and per-system field, read them back singly, as a fused
    window in arbitrary order, and through a loader: values, levels and per-sample metadata survive."""
    from nvalchemi_toolkit_b200.data.datapipes import DataLoader, Dataset
    from nvalchemi_toolkit_b200.data.zarr_store import (AtomicDataZarrReader, AtomicDataZarrWriter, ZarrArrayConfig,
                                                        ZarrWriteConfig)

    g = torch.Generator().manual_seed(seed)
    data = []
    for i, n in enumerate(sizes):
        d = random_molecule(n, seed + i, n_edges=edges)
        d.add_node_property("magmom", torch.randn(n, 2, generator=g))
        with pytest.raises(ValueError, match="already a system-level field"):
            d.add_node_property("spin", torch.zeros(n, 1))      # the built-in per-system total spin owns that name
        d.add_system_property("tag", torch.tensor([[float(i)]]))
        if edges:
            d.add_edge_property("bond_order", torch.rand(edges, 1, generator=g))
        data.append(d)
    cfg = ZarrArrayConfig(chunk_rows=chunk, compressor=compressor)
    path = tmp_path_factory.mktemp("ds") / "s.zarr"
    AtomicDataZarrWriter(path, config=ZarrWriteConfig(core=cfg, meta=cfg, custom=cfg)).write(data)
    reader = AtomicDataZarrReader(path)
    assert len(reader) == len(sizes)
    assert [reader.get_metadata(i) for i in range(len(sizes))] == [(n, edges) for n in sizes]
    ds = Dataset(reader, num_workers=1)
    order = torch.randperm(len(sizes), generator=g).tolist()
    window = ds.fetch(order).result()
    for (item, meta), i in zip(window, order):
        ref = data[i]
        assert torch.equal(item.positions, ref.positions) and torch.equal(item.atomic_numbers, ref.atomic_numbers)
        assert torch.equal(item.magmom, ref.magmom) and item.level_of("magmom") == "node"
        assert float(item.tag) == float(i) and item.level_of("tag") == "system"
        if edges:
            assert torch.equal(item.neighbor_list, ref.neighbor_list)
            assert torch.equal(item.bond_order, ref.bond_order) and item.level_of("bond_order") == "edge"
    single, _ = ds[order[0]]
    assert torch.equal(single.magmom, data[order[0]].magmom)
    batches = list(DataLoader(ds, batch_size=2))
    assert sum(b.num_graphs for b in batches) == len(sizes)
    assert torch.equal(torch.cat([b.tag.reshape(-1) for b in batches]), torch.arange(len(sizes), dtype=torch.float32))
    assert torch.equal(torch.cat([b.magmom for b in batches]), torch.cat([d.magmom for d in data]))
    ds.close()
