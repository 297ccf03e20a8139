"""Per-layer ghost refresh of unmodified message-passing models (``distributed/dispatch.py``), storage policies and
operator adapters.  Multi-rank cases run as gloo processes on CPU."""
import os

import pytest
import torch
import torch.distributed as dist

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.distributed import DistributedModel, DomainConfig, ShardedBatch, ShardTensor
from nvalchemi_toolkit_b200.distributed.dispatch import (AdapterRegistry, FunctionAdapter, HaloDispatchMode, OpAdapter,
                                                         current_dispatch)
from nvalchemi_toolkit_b200.distributed.storage_policy import (GraphParallelPolicy, HaloStoragePolicy, PlainShard,
                                                               RefreshOnlyHaloPolicy, policy_from_dict, policy_to_dict,
                                                               row_offsets)
from tests.helpers import fcc_supercell
from tests.test_distributed_api import _mace_model, _reference


def test_policy_round_trip_and_offsets():
    for p in (PlainShard(), HaloStoragePolicy(), HaloStoragePolicy("local", "halo_read"), RefreshOnlyHaloPolicy(),
              GraphParallelPolicy()):
        q = policy_from_dict(policy_to_dict(p))
        assert type(q) is type(p) and q == p
    assert row_offsets([3, 0, 2]) == [0, 3, 3, 5]
    with pytest.raises(ValueError):
        HaloStoragePolicy(scatter_mode="nope")
    with pytest.raises(ValueError):
        policy_from_dict({"kind": "unknown"})
    assert RefreshOnlyHaloPolicy().partition_mode == "halo" and GraphParallelPolicy().partition_mode == "graph_partition"


class _FakeHalo:
    """Two 'ranks' in one process: ghost rows are copies of chosen owned rows (periodic self-images)."""

    def __init__(self, src_rows):
        self.src = torch.as_tensor(src_rows)
        self.n_ghost = len(src_rows)

    def forward(self, owned):
        return owned[self.src]

    def reverse_add(self, ghost_vals, owned):
        owned.index_add_(0, self.src, ghost_vals)
        return owned


def test_mode_tracks_staleness_and_refreshes_before_gather():
    halo = _FakeHalo([0, 2])
    n_owned = 4
    h = torch.arange(6.0).reshape(6, 1).requires_grad_()
    src, dst = torch.tensor([4, 5, 1]), torch.tensor([0, 1, 2])
    with HaloDispatchMode(halo, n_owned) as mode:
        assert current_dispatch() is mode
        agg = torch.zeros(6, 1).index_add_(0, dst, h[src])     # fresh gather, scatter marks the result stale
        assert mode.is_stale(agg) and mode.stats["refreshes"] == 0
        y = torch.tanh(agg) * 2.0                                # staleness propagates through row-wise ops
        assert mode.is_stale(y)
        g = y[src]                                               # ghost rows 4, 5 are refreshed from rows 0, 2 first
        assert mode.stats["refreshes"] == 1
        assert torch.allclose(g, torch.stack([y[0], y[2], y[1]]).detach())
        _ = y.index_select(0, dst)                               # same stale tensor again: cached refresh
        assert mode.stats["refreshes"] == 1
        per_system = torch.zeros(1, 1).index_add_(0, torch.zeros(6, dtype=torch.long), y)  # owned rows only
        assert mode.stats["masked_reductions"] == 1
        assert torch.allclose(per_system, y[:4].sum(0, keepdim=True))
        g.sum().backward()                                       # ghost-row gradients flow back to their owners
    assert current_dispatch() is None
    assert h.grad is not None and torch.isfinite(h.grad).all()


def test_fold_policy_returns_ghost_partials_to_owners():
    halo = _FakeHalo([0, 2])
    with HaloDispatchMode(halo, 4, HaloStoragePolicy()) as mode:
        out = torch.zeros(6, 1)
        out.index_add_(0, torch.tensor([4, 5, 1]), torch.tensor([[1.0], [2.0], [3.0]]))
        assert mode.stats["folds"] == 1 and mode.is_stale(out)
    assert out.flatten().tolist() == [1.0, 3.0, 2.0, 0.0, 0.0, 0.0]


def _fused_layer(h, src, dst):
    """An operator the mode cannot see into once wrapped (stands for a fused gather+scatter kernel)."""
    return torch.zeros_like(h).index_add_(0, dst, h[src].detach())


def test_adapter_refreshes_inputs_and_marks_outputs():
    import sys

    me = sys.modules[__name__]
    halo = _FakeHalo([0, 2])
    src, dst = torch.tensor([4, 5, 1]), torch.tensor([0, 1, 2])
    registry = AdapterRegistry([FunctionAdapter(me, "_fused_layer", node_inputs=(0,), node_outputs=(0,))])
    h = torch.arange(6.0).reshape(6, 1)
    with registry, HaloDispatchMode(halo, 4) as mode:
        with torch._C.DisableTorchFunction():
            a = torch.zeros(6, 1).index_add_(0, dst, h[src])
        mode.mark_stale(a)
        b = me._fused_layer(a, src, dst)
        assert mode.stats["refreshes"] == 1 and mode.is_stale(b)
        assert float(b[0]) == float(a[0]) and float(b[1]) == float(a[2])  # rows 4, 5 were read as copies of rows 0, 2
    assert not hasattr(me._fused_layer, "__wrapped_by_adapter__")  # restored
    assert OpAdapter().wrap(lambda x: x + 1)(1) == 2             # outside a distributed forward: plain call


class _MPNN(torch.nn.Module):
    """Three message-passing layers written with plain gathers and scatters; knows nothing about decomposition."""

    def __init__(self, width=8, layers=3):
        super().__init__()
        self.emb = torch.nn.Embedding(100, width)
        self.mix = torch.nn.ModuleList(torch.nn.Linear(width, width) for _ in range(layers))
        self.out = torch.nn.Linear(width, 1)

    def forward(self, z, pos, src, dst, shifts, batch, n_graphs):
        h = self.emb(z)
        d = (pos[src] + shifts - pos[dst]).norm(dim=-1, keepdim=True)
        w = torch.exp(-d) * (d < 3.0)
        for lin in self.mix:
            m = lin(h)[src] * w
            h = h + torch.tanh(torch.zeros_like(h).index_add_(0, dst, m))
        e = self.out(h).squeeze(-1)
        return torch.zeros(n_graphs, dtype=pos.dtype).index_add_(0, batch, e)


def _mpnn_wrapper():
    from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec
    from nvalchemi_toolkit_b200.models.base import BaseModelMixin, ModelConfig, NeighborConfig, NeighborListFormat

    class Wrapper(torch.nn.Module, BaseModelMixin):
        def __init__(self):
            super().__init__()
            torch.manual_seed(3)
            self.net = _MPNN().double()
            self.model_config = ModelConfig(outputs=frozenset({"energy", "forces"}),
                                            neighbor_config=NeighborConfig(cutoff=3.0, format=NeighborListFormat.MATRIX))

        def forward(self, data, **kw):
            pos = data.positions.detach().requires_grad_()
            nm, num = data.neighbor_matrix.long(), data.num_neighbors.long()
            k = torch.arange(nm.shape[1])
            valid = k[None, :] < num[:, None]
            dst = torch.arange(nm.shape[0])[:, None].expand_as(nm)[valid]
            src = nm[valid]
            S = data.neighbor_matrix_shifts[valid].to(pos.dtype)
            cell = data.cell[data.batch_idx.long()[dst]].to(pos.dtype)
            shifts = torch.einsum("ei,eij->ej", S, cell)
            ng = int(data.cell.shape[0])
            e = self.net(data.atomic_numbers.long(), pos, src, dst, shifts, data.batch_idx.long(), ng)
            (g,) = torch.autograd.grad(e.sum(), pos)
            return {"energy": e.detach().reshape(ng, 1), "forces": -g}

        def distribution_spec(self, strategy=None):
            return MLIPSpec("test_mpnn", message_passes=3, consolidation=Consolidation.WEIGHTED_ENERGY,
                            refresh_per_layer=True)

    return Wrapper()


def _worker(rank, world, port, q, which):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
        cfg = DomainConfig(cutoff=3.0, skin=0.0)
        if which == "mace":
            model = _mace_model()
            model.model_config.active_outputs = {"energy", "forces"}
            spec = model.distribution_spec().with_(refresh_per_layer=True)
            deep = ShardedBatch.from_batch(batch, cfg, model.distribution_spec()).n_ghost
        else:
            model = _mpnn_wrapper()
            spec = model.distribution_spec()
            if which == "mpnn_fold":  # every edge on its sender's owner; partial sums of ghost receivers are folded
                spec = spec.with_(storage_policy={"kind": "halo"})
            deep = ShardedBatch.from_batch(batch, cfg, spec.with_(refresh_per_layer=False)).n_ghost
        sh = ShardedBatch.from_batch(batch, cfg, spec)
        dm = DistributedModel(model, cfg, spec=spec)
        out = dm(sh)
        forces = ShardTensor(out["forces"], sh).full_tensor()
        q.put((rank, forces.tolist(), out["energy"].reshape(-1).tolist(), sh.n_ghost, deep, dm.last_dispatch_stats))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("which,port", [("mpnn", 29671), ("mace", 29673), ("mpnn_fold", 29675)])
def test_unmodified_model_with_one_cutoff_halo_matches_single_process(which, port):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, which)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        item = q.get(timeout=240)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
    model = _mace_model() if which == "mace" else _mpnn_wrapper()
    model.model_config.active_outputs = {"energy", "forces"}
    ref = _reference(model, batch)
    for r in range(2):
        forces, energy, n_ghost, n_ghost_deep, stats = res[r]
        assert torch.allclose(torch.tensor(forces, dtype=torch.float64), ref["forces"], atol=1e-8)
        assert abs(energy[0] - float(ref["energy"].detach().reshape(-1)[0])) < 1e-8
        assert 0 < n_ghost < n_ghost_deep           # one cutoff of ghosts instead of one per message pass
        assert stats["refreshes"] >= 1              # ghost feature rows were exchanged between the layers
        assert (stats["folds"] >= 3) == (which == "mpnn_fold")


def _p2p_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nvalchemi_toolkit_b200.distributed import halo as halo_mod
        from nvalchemi_toolkit_b200.distributed._runtime import mesh_group

        torch.set_num_threads(1)
        # rank r sends r + p + 1 rows to peer p, except nothing to its right neighbour (an empty split)
        send = [0 if p == (rank + 1) % world else rank + p + 1 for p in range(world)]
        recv = halo_mod.exchange_counts(send, torch.device("cpu"))
        rows = torch.arange(sum(send), dtype=torch.float64)[:, None] + 100.0 * rank
        a = halo_mod.all_to_all_rows(rows, send, recv)
        b = halo_mod.neighbor_exchange_rows(rows, send, recv)
        same = torch.equal(a, b)
        halo_mod.TRANSPORT = "p2p"   # the whole distributed evaluation over point-to-point messages
        batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
        cfg = DomainConfig(cutoff=3.0, skin=0.0)
        model = _mpnn_wrapper()
        spec = model.distribution_spec()
        sh = ShardedBatch.from_batch(batch, cfg, spec)
        out = DistributedModel(model, cfg, spec=spec)(sh)
        forces = ShardTensor(out["forces"], sh).full_tensor()
        q.put((rank, same, forces.tolist(), mesh_group(None) is None, mesh_group(dist.group.WORLD) is dist.group.WORLD))
    finally:
        dist.destroy_process_group()


def test_neighbor_only_p2p_transport_matches_all_to_all():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_p2p_worker, args=(r, 3, 29677, q)) for r in range(3)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(3):
        item = q.get(timeout=240)
        res[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    batch = Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])
    ref = _reference(_mpnn_wrapper(), batch)
    for r in range(3):
        same, forces, g0, g1 = res[r]
        assert same and g0 and g1
        assert torch.allclose(torch.tensor(forces, dtype=torch.float64), ref["forces"], atol=1e-8)


def _batch_factory():
    return Batch.from_data_list([fcc_supercell(4, a=3.61, z=29, noise=0.08, seed=3, dtype=torch.float64)])


def _shallow_spec_mpnn():
    """The three-layer network declared with a ONE-hop halo and no per-layer refresh: wrong from the second layer on."""
    m = _mpnn_wrapper()
    spec = m.distribution_spec().with_(refresh_per_layer=False, message_passes=1)
    m.distribution_spec = lambda strategy=None: spec
    return m


def test_layer_diff_locates_the_first_deviating_layer():
    from nvalchemi_toolkit_b200.distributed.validate import layer_diff

    good = layer_diff(_mpnn_wrapper, _batch_factory, 2, cutoff=3.0, port=29681)
    assert good and all(r["ok"] for r in good)
    bad = layer_diff(_shallow_spec_mpnn, _batch_factory, 2, cutoff=3.0, port=29683)
    by_name = {r["module"]: r["ok"] for r in bad}
    assert by_name["net.emb"] and by_name["net.mix.0"]        # inputs of the first aggregation are still exact
    assert not by_name["net.mix.2"] and not by_name["net.out"]  # stale ghost rows have reached the owned atoms


def _undeclared_mpnn():
    m = _mpnn_wrapper()
    m.distribution_spec = lambda strategy=None: None
    return m


def test_spec_inferred_from_a_trace_counts_message_passes_and_validates():
    """No declared spec: the trace of one single-process forward counts three neighbour aggregations on the way to the
    energy, sees the model differentiate internally, and the spec built from that reproduces the forces on two ranks."""
    from nvalchemi_toolkit_b200.distributed.infer_spec import infer_spec
    from nvalchemi_toolkit_b200.distributed.spec import Consolidation, MLIPSpec
    from nvalchemi_toolkit_b200.distributed.validate import trace_and_validate

    spec, summary = infer_spec(_undeclared_mpnn(), _batch_factory())
    assert spec.message_passes == 3 and summary.node_scatters == 3 and summary.system_reductions == 1
    assert summary.deep_gathers == 2 and summary.used_autograd           # layers 2 and 3 read aggregated features
    assert spec.consolidation == Consolidation.WEIGHTED_ENERGY and spec.node_outputs == ("forces",)
    assert spec.extensive_outputs == ("energy",)
    # a declared field wins over the trace, the rest is filled in
    prior = MLIPSpec("mine", refresh_per_layer=True)
    merged, _ = infer_spec(_undeclared_mpnn(), _batch_factory(), prior=prior)
    assert merged.name == "mine" and merged.refresh_per_layer and merged.message_passes == 3
    assert spec.refresh_per_layer and "owned-only reductions" in spec.notes  # the model sums over atoms itself
    rep = trace_and_validate(_undeclared_mpnn, _batch_factory, 2, cutoff=3.0, port=29687, atol=1e-8)
    assert rep.ok and rep.attempts[0]["label"] == "inferred spec" and "3 message pass" in rep.trace
    assert "inferred spec" in rep.next_action and MLIPSpec.from_dict(rep.spec_dict()).message_passes == 3


def test_opaque_neighbour_operator_is_given_one_message_pass():
    from nvalchemi_toolkit_b200.distributed.infer_spec import infer_spec
    from nvalchemi_toolkit_b200.models.lj import LennardJonesModelWrapper
    from tests.helpers import fcc_supercell

    model = LennardJonesModelWrapper(epsilon=0.01, sigma=2.3, cutoff=5.0)
    batch = Batch.from_data_list([fcc_supercell(3, a=3.61, z=29, noise=0.05, seed=1)])
    spec, summary = infer_spec(model, batch)
    assert spec.message_passes == 1 and "opaque operator" in spec.notes and "energy" in spec.extensive_outputs


@torch.jit.script
def _scripted_sum(x: torch.Tensor, idx: torch.Tensor, n: int) -> torch.Tensor:
    return torch.zeros(n, x.shape[1], dtype=x.dtype).index_add_(0, idx, x)


def test_scripted_code_is_reported_with_the_adapter_to_declare():
    from nvalchemi_toolkit_b200.distributed.validate import ScriptedOpReport, detect_scripted_ops

    class Plain(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(2, 2)

    class WithScriptedBlock(Plain):
        def __init__(self):
            super().__init__()
            self.block = torch.jit.script(torch.nn.Sequential(torch.nn.Linear(2, 2), torch.nn.Tanh()))

    rep = detect_scripted_ops(WithScriptedBlock())
    assert isinstance(rep, ScriptedOpReport) and rep.found and rep.modules[0] == "block"
    assert any(f.endswith("test_dispatch_refresh._scripted_sum") for f in rep.functions)   # defined beside the model class
    assert "JitAdapter" in rep.advice() and "ModuleForwardAdapter" in rep.advice()
    clean = detect_scripted_ops(torch.nn.Linear(2, 2))
    assert not clean.found and "no scripted code" in clean.advice()
    assert not detect_scripted_ops(object()).found
