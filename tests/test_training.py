# SPDX-License-Identifier: Apache-2.0
"""Training loop: stage order, losses, update hooks, checkpoints/resume, data-parallel gradient all-reduce (gloo)."""
import os

import pytest
import torch

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.models import DemoModelWrapper
from nvalchemi_toolkit_b200.training import (ComposedLossFunction, EnergyMSELoss, ForceMSELoss, LinearWeight,
                                             OptimizerConfig, TrainingStage, TrainingStrategy, ValidationConfig)
from nvalchemi_toolkit_b200.training.hooks import (CheckpointHook, EMAHook, FusedGradAllReduceHook,
                                                   GradientAccumulationHook, GradientClipHook, LossSpikeSkipHook,
                                                   TrainableParameterHook)
from tests.helpers import random_molecule


def _dataset(n=12, seed=0):
    torch.manual_seed(seed)
    teacher = DemoModelWrapper()
    out = []
    for i in range(n):
        d = random_molecule(6 + i % 3, seed * 100 + i)
        b = Batch.from_data_list([d])
        o = teacher(b)
        d.__dict__["energy"] = o["energy"].detach().reshape(1, 1)
        d.__dict__["forces"] = o["forces"].detach()
        out.append(d)
    return out


def _loader(data, bs=4):
    return [Batch.from_data_list(data[i:i + bs]) for i in range(0, len(data), bs)]


def _strategy(**kw):
    torch.manual_seed(1)
    loss = EnergyMSELoss() + 10.0 * ForceMSELoss()
    if "num_steps" not in kw:
        kw.setdefault("num_epochs", 2)
    kw.setdefault("devices", ["cpu"])
    return TrainingStrategy(DemoModelWrapper(), OptimizerConfig(kwargs={"lr": 3e-3}), loss, **kw)


class Recorder:
    frequency = 1

    def __init__(self):
        self.stage, self.seen = None, []

    def _runs_on_stage(self, stage):
        return stage not in (TrainingStage.DO_BACKWARD, TrainingStage.DO_OPTIMIZER_STEP)

    def __call__(self, ctx, stage):
        self.seen.append(stage)


def test_loss_decreases_and_stage_order():
    rec = Recorder()
    st = _strategy(num_epochs=15, hooks=[rec, GradientClipHook(5.0)])
    loader = _loader(_dataset())
    st.train_batch(loader[0])
    first = float(st.last_losses["total_loss"])
    per_batch = [s for s in rec.seen if s not in (TrainingStage.SETUP,)]
    names = [s.name for s in per_batch]
    assert names == ["BEFORE_BATCH", "BEFORE_FORWARD", "AFTER_FORWARD", "BEFORE_LOSS", "AFTER_LOSS", "BEFORE_BACKWARD",
                     "AFTER_BACKWARD", "BEFORE_OPTIMIZER_STEP", "AFTER_OPTIMIZER_STEP", "AFTER_BATCH"]
    st.run(loader)
    assert float(st.last_losses["total_loss"]) < 0.5 * first
    assert st.epoch_count == 15 and st.step_count == 15 * 3  # the manual batch counted as the first of epoch 0


def test_loss_composition_and_schedules():
    l = EnergyMSELoss(weight=LinearWeight(0.0, 1.0, 10)) + 2.0 * ForceMSELoss()
    assert isinstance(l, ComposedLossFunction) and len(l.terms) == 2
    assert l.terms[0].weight_at(5, 0) == pytest.approx(0.5) and l.terms[1].weight_at(0, 0) == 2.0
    spec = l.to_spec()
    l2 = ComposedLossFunction.from_spec(spec)
    assert l2.terms[0].weight_at(10, 0) == pytest.approx(1.0) and l2.required_predictions() == {"energy", "forces"}


def test_accumulation_and_spike_skip():
    st = _strategy(num_steps=4, hooks=[GradientAccumulationHook(2), LossSpikeSkipHook(factor=1e9)])
    loader = _loader(_dataset(), bs=2)
    st.run(loader)
    assert st.step_count == 4 and st.batch_count == 8


def test_checkpoint_resume_reproduces_run(tmp_path):
    data = _dataset()
    loader = _loader(data)
    ref = _strategy(num_epochs=2, hooks=[EMAHook(decay=0.9)])
    ref.run(loader)
    a = _strategy(num_epochs=1, hooks=[EMAHook(decay=0.9), CheckpointHook(tmp_path / "ck", every_n_epochs=1)])
    a.run(loader)
    assert (tmp_path / "ck" / "manifest.json").exists() and (tmp_path / "ck" / "models" / "main" / "spec.json").exists()
    b = _strategy(num_epochs=2, hooks=[EMAHook(decay=0.9)])
    b.load_checkpoint(tmp_path / "ck")
    assert b.epoch_count == 1 and b.step_count == 3
    b.run(loader)
    for p, q in zip(ref.models["main"].parameters(), b.models["main"].parameters()):
        assert torch.allclose(p, q, atol=1e-6)
    assert b.step_count == ref.step_count == 6


def test_validation_and_trainable_filter():
    data = _dataset()
    st = _strategy(num_epochs=1, validation_config=ValidationConfig(data=_loader(data[:4]), every_n_epochs=1),
                   hooks=[TrainableParameterHook([r"projection"])])
    st.run(_loader(data))
    assert st.last_validation is not None and "total_loss" in st.last_validation and st.last_validation["num_graphs"] == 4
    frozen = [n for n, p in st.models["main"].named_parameters() if not p.requires_grad]
    assert frozen and all("projection" not in n for n in frozen)


def _dp_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        data = _dataset(8)
        st = _strategy(num_steps=3, hooks=[FusedGradAllReduceHook()])
        for step in range(3):  # rank r, step s: graphs [4 (s % 2) + 2 r, +2): equal counts per rank
            lo = 4 * (step % 2) + 2 * rank
            st.train_batch(Batch.from_data_list(data[lo: lo + 2]))
        q.put((rank, [p.detach().reshape(-1).tolist() for p in st.models["main"].parameters()]))
    finally:
        dist.destroy_process_group()


def _dp_accum_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist

    from nvalchemi_toolkit_b200.training.hooks.library import GradientAccumulationHook

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        data = _dataset(8)
        hook = FusedGradAllReduceHook()
        calls = []
        orig = dist.all_reduce

        def spy(t, *a, **k):
            calls.append(int(t.numel()))
            return orig(t, *a, **k)

        dist.all_reduce = spy
        st = _strategy(num_steps=2, hooks=[GradientAccumulationHook(steps=2), hook])
        for micro in range(4):  # optimiser step s = micro // 2 sees graphs [4 (s % 2), +4); rank r takes one per micro-batch
            lo = 4 * ((micro // 2) % 2) + 2 * (micro % 2) + rank
            st.train_batch(Batch.from_data_list(data[lo: lo + 1]))
        dist.all_reduce = orig
        big = [c for c in calls if c > 8]
        q.put((rank, st.step_count, len(big), [p.detach().reshape(-1).tolist() for p in st.models["main"].parameters()]))
    finally:
        dist.destroy_process_group()


def test_gradient_accumulation_reduces_once_per_optimizer_step():
    """With accumulation the cross-rank reduction runs with the LAST micro-batch of an optimiser step (once per step, on the
    accumulated gradients), and the replicas stay in lock-step."""
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_accum_worker, args=(r, 2, 29589, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = {r[0]: r[1:] for r in (q.get(timeout=120) for _ in range(2))}
    for p in procs:
        p.join(timeout=30)
    assert res[0][0] == res[1][0] == 2 and res[0][1] == res[1][1] == 2  # two optimiser steps, two gradient reductions
    for a, b in zip(res[0][2], res[1][2]):
        assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=1e-7)


def test_fused_gradient_allreduce_matches_single_process():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, 29588, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    for a, b in zip(res[0], res[1]):
        assert torch.allclose(torch.tensor(a), torch.tensor(b), atol=1e-7)  # ranks stay in lock-step
    data = _dataset(8)
    st = _strategy(num_steps=3)
    for step in range(3):
        st.train_batch(Batch.from_data_list(data[4 * (step % 2): 4 * (step % 2) + 4]))
    for a, b in zip(res[0], st.models["main"].parameters()):
        assert torch.allclose(torch.tensor(a), b.detach().reshape(-1), atol=5e-3)  # Adam amplifies rounding of tiny gradients


def test_checkpoint_layout_matches_reference_and_reads_a_reference_fixture(tmp_path):
    """Field names and paths of the reference's layout: ``checkpoint_index`` / ``associations`` in the manifest, named
    optimizer / scheduler components, ``hooks/checkpoints/N.pt``, ``strategy.json`` + ``strategy/checkpoints/N.json``."""
    import json

    from nvalchemi_toolkit_b200.training import checkpoint as ckpt

    a = _strategy(num_epochs=1, hooks=[EMAHook(decay=0.9), CheckpointHook(tmp_path / "ck", every_n_epochs=1)])
    a.run(_loader(_dataset()))
    root = tmp_path / "ck"
    man = json.loads((root / "manifest.json").read_text())
    assert set(man) == {"schema_version", "checkpoint_index", "models", "optimizers", "schedulers", "associations"}
    assert man["checkpoint_index"] == 0 and man["models"] == ["main"] and man["optimizers"] == ["main_optimizer"]
    assoc = man["associations"]["main"]
    assert assoc["optimizers"] == ["main_optimizer"] and assoc["optimizer_parameter_names"]["main_optimizer"]
    spec = json.loads((root / "models" / "main" / "spec.json").read_text())
    assert "cls_path" in spec and "timestamp" in spec
    assert (root / "optimizers" / "main_optimizer" / "checkpoints" / "0.pt").exists()
    assert (root / "hooks" / "checkpoints" / "0.pt").exists()
    assert (root / "strategy.json").exists() and (root / "strategy" / "checkpoints" / "0.json").exists()
    hook_states = torch.load(root / "hooks" / "checkpoints" / "0.pt", weights_only=True)  # no pickle-dependent objects
    assert list(hook_states) == [f"{EMAHook.__module__}.EMAHook:0"]
    assert ckpt.validate_checkpoint(root) == []

    # a directory written by hand exactly as the reference lays it out
    fix = tmp_path / "ref"
    model = a.models["main"]
    opt = a._optimizers[0]
    for kind, name, state in (("models", "main", model.state_dict()), ("optimizers", "main_optimizer", opt.state_dict())):
        d = fix / kind / name / "checkpoints"
        d.mkdir(parents=True)
        (fix / kind / name / "spec.json").write_text(json.dumps({"cls_path": "torch.nn.Linear", "timestamp": "2026-01-01T00:00:00+00:00"}))
        torch.save(state, d / "3.pt")
    (fix / "hooks" / "checkpoints").mkdir(parents=True)
    torch.save({f"{EMAHook.__module__}.EMAHook:0": {"num_updates": 5, "ema": None}}, fix / "hooks" / "checkpoints" / "3.pt")
    meta = {"step_count": 7, "global_step_count": 7, "batch_count": 7, "epoch_count": 2, "epoch_step_count": 1}
    (fix / "strategy.json").write_text(json.dumps(meta))
    (fix / "strategy" / "checkpoints").mkdir(parents=True)
    (fix / "strategy" / "checkpoints" / "3.json").write_text(json.dumps(meta))
    (fix / "manifest.json").write_text(json.dumps({
        "schema_version": 1, "checkpoint_index": 3, "models": ["main"], "optimizers": ["main_optimizer"], "schedulers": [],
        "associations": {"main": {"optimizers": ["main_optimizer"], "schedulers": []}}}))
    b = _strategy(num_epochs=3, hooks=[EMAHook(decay=0.9)])
    b.load_checkpoint(fix)
    assert (b.step_count, b.epoch_count, b.epoch_step_count) == (7, 2, 1)
    b._setup(_loader(_dataset()))
    for p, q in zip(model.parameters(), b.models["main"].parameters()):
        assert torch.equal(p.detach().cpu(), q.detach().cpu())
    assert b.hooks[0].num_updates == 5 or any(getattr(h, "num_updates", None) == 5 for h in b.hooks)
    assert ckpt.validate_checkpoint(fix) == []
    (fix / "manifest.json").write_text(json.dumps({"schema_version": 1, "models": ["main"]}))
    with pytest.raises(ValueError):
        ckpt.CheckpointManifest(fix)


def test_asynchronous_checkpoint_holds_the_snapshot_not_the_live_weights(tmp_path):
    """``save_checkpoint(asynchronous=True)`` returns before the files exist; what lands on disk is the state at the call,
    even when the parameters change while the writer runs; the next index appears only after ``wait()``."""
    from nvalchemi_toolkit_b200.training import checkpoint as ck

    net = torch.nn.Linear(4, 3)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    net(torch.randn(2, 4)).sum().backward()
    opt.step()
    want = {k: v.clone() for k, v in net.state_dict().items()}
    handle = ck.save_checkpoint(tmp_path, 7, {"main": net}, [opt], [None], [], {"step_count": 7}, asynchronous=True)
    with torch.no_grad():
        for p in net.parameters():
            p.add_(100.0)  # training goes on
    assert handle.wait() == tmp_path and handle.done()
    assert ck.CheckpointManifest(tmp_path).checkpoint_index == 0 and not ck.validate_checkpoint(tmp_path)
    fresh = torch.nn.Linear(4, 3)
    ck.load_checkpoint(tmp_path, {"main": fresh})
    for k, v in fresh.state_dict().items():
        assert torch.equal(v, want[k])
    # a failing writer surfaces in wait()
    bad = ck.save_checkpoint(tmp_path, 8, {"main": torch.nn.Embedding(5, 3)}, [], [], [], {}, asynchronous=True)
    with pytest.raises(ValueError, match="spec.json disagrees"):
        bad.wait()


def test_validation_loop_restores_gradients_and_supports_metrics_and_own_loss():
    from nvalchemi_toolkit_b200.training.validation import ValidationConfig, ValidationLoop, ensure_reiterable

    data = _dataset(8)
    st = _strategy(num_steps=1)
    st.train_batch(Batch.from_data_list(data[:4]))
    model = st.models["main"]
    grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    assert grads and model.training
    seen = []
    cfg = ValidationConfig(data=_loader(data[4:]), loss_fn=EnergyMSELoss(weight=1.0) + ForceMSELoss(weight=0.0),
                           metrics={"energy_mae": lambda pred, b: (pred["energy"].reshape(-1) - b.energy.reshape(-1)).abs().mean()},
                           batch_callback=lambda b, p, l: seen.append(b.num_graphs))
    out = ValidationLoop.from_training_strategy(st, cfg).execute()
    assert out["num_graphs"] == 4 and out["num_batches"] == len(seen) and "metric/energy_mae" in out and out["step"] == 1
    assert abs(out["total_loss"] - out[[k for k in out if k.startswith("EnergyMSE")][0]]) < 1e-9  # forces weigh nothing here
    assert model.training
    for n, p in model.named_parameters():
        if n in grads:
            assert torch.equal(p.grad, grads[n])
    with pytest.raises(TypeError, match="re-iterable"):
        ValidationConfig(data=iter(_loader(data)))
    with pytest.raises(ValueError, match="every_n_steps"):
        ValidationConfig(every_n_steps=0)
    assert ensure_reiterable([1, 2]) == [1, 2]


def test_optimizer_config_checks_kwargs_and_builds_parameter_groups():
    from nvalchemi_toolkit_b200.training.optimizers import OptimizerConfig, ParamGroupSpec, setup_optimizers, step_schedulers

    with pytest.raises(ValueError, match="weight_decy"):
        OptimizerConfig(cls=torch.optim.AdamW, kwargs={"lr": 1e-3, "weight_decy": 0.1})
    with pytest.raises(ValueError, match="scheduler"):
        OptimizerConfig(scheduler_cls=torch.optim.lr_scheduler.StepLR, scheduler_kwargs={"step_sz": 3})
    with pytest.raises(ValueError, match="scheduler_interval"):
        OptimizerConfig(scheduler_interval="sometimes")
    net = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.LayerNorm(8), torch.nn.Linear(8, 1))
    cfg = OptimizerConfig(cls="torch.optim.AdamW", kwargs={"lr": 1e-3, "weight_decay": 0.1},
                          param_groups=[ParamGroupSpec(pattern=r"bias$|\.1\.", options={"weight_decay": 0.0}),
                                        ParamGroupSpec(pattern=r"\.2\.weight", options={"lr": 1e-4})],
                          scheduler_cls=torch.optim.lr_scheduler.ReduceLROnPlateau, scheduler_kwargs={"patience": 0, "factor": 0.5},
                          scheduler_interval="validation", scheduler_metric_adapter=lambda m: m["a"] + m["b"])
    opts, scheds, keys = setup_optimizers({"main": net}, {"main": [cfg]})
    groups = opts[0].param_groups
    assert keys == ["main"] and len(groups) == 3
    assert [g["weight_decay"] for g in groups] == [0.1, 0.0, 0.1] and [g["lr"] for g in groups] == [1e-3, 1e-3, 1e-4]
    assert sum(len(g["params"]) for g in groups) == 6 and len(groups[1]["params"]) == 4  # three biases + the norm weight
    step_schedulers(scheds, [cfg], "validation", {"a": 1.0, "b": 1.0})
    step_schedulers(scheds, [cfg], "validation", {"a": 2.0, "b": 1.0})  # worse: the plateau scheduler halves every lr
    assert [g["lr"] for g in opts[0].param_groups] == [5e-4, 5e-4, 5e-5]
    assert cfg.to_spec()["param_groups"][0]["options"] == {"weight_decay": 0.0}


def test_finetune_from_pretrained_checkpoint_inherits_weights_only(tmp_path):
    """A new fine-tuning run from a checkpoint directory: models rebuilt from their specs with the saved weights, loss and
    optimiser classes optionally reused (with the fine-tuning learning rate), counters and optimiser state fresh."""
    from nvalchemi_toolkit_b200.training.finetune import DEFAULT_FINETUNE_LR, FineTuningStrategy

    data = _dataset(8)
    st = _strategy(num_steps=3)
    st.run(_loader(data))
    st.save_checkpoint(tmp_path / "src")
    ft = FineTuningStrategy.from_pretrained_checkpoint(tmp_path / "src", use_original_loss=True, use_original_opt_class=True,
                                                       trainable=[r"projection"], num_steps=2, devices=["cpu"])
    assert ft.step_count == 0 and ft.num_steps == 2
    for (n, a), (_, b) in zip(st.models["main"].state_dict().items(), ft.models["main"].state_dict().items()):
        assert torch.equal(a, b), n
    cfg = ft.optimizer_configs["main"][0]
    assert cfg.kwargs["lr"] == DEFAULT_FINETUNE_LR and type(ft.loss_fn).__name__ == type(st.loss_fn).__name__
    before = {n: p.detach().clone() for n, p in ft.models["main"].named_parameters()}
    ft.run(_loader(data))
    named = dict(ft.models["main"].named_parameters())
    changed = [n for n, p in named.items() if not torch.equal(p, before[n])]
    # the optimiser moves the projection only; the embedding table renormalises its rows in the forward pass (max_norm)
    assert "model.projection.weight" in changed and set(changed) <= {"model.projection.weight", "model.embedding.weight"}
    assert all(not named[n].requires_grad for n in named if "projection" not in n) and ft.step_count == 2
    assert [len(g["params"]) for o in ft._optimizers for g in o.param_groups] == [1]
    with pytest.raises(ValueError, match="optimiser"):
        import json

        meta = json.loads((tmp_path / "src" / "strategy.json").read_text())
        meta["spec"]["optimizer_configs"] = {}
        (tmp_path / "src" / "strategy.json").write_text(json.dumps(meta))
        idx_file = sorted((tmp_path / "src" / "strategy" / "checkpoints").glob("*.json"))[-1]
        idx_file.write_text(json.dumps(meta))
        FineTuningStrategy.from_pretrained_checkpoint(tmp_path / "src", use_original_opt_class=True, num_steps=1, devices=["cpu"])


class _Labels:
    """Minimal stand-in for a batch: the attributes the loss terms read."""

    def __init__(self, **fields):
        self.__dict__.update(fields)

    def keys(self):
        return list(self.__dict__)


def _mixed_batch():
    return _Labels(num_graphs=3, batch_idx=torch.tensor([0, 0, 1, 1, 1, 2]), num_nodes_per_graph=torch.tensor([2, 3, 1]),
                   energy=torch.tensor([1.0, float("nan"), 3.0]),
                   forces=torch.arange(18, dtype=torch.float32).reshape(6, 3) / 10)


def test_loss_terms_skip_missing_labels_in_value_and_gradient():
    from nvalchemi_toolkit_b200.training.losses import EnergyMSELoss, ForceL2NormLoss, ForceMSELoss

    b = _mixed_batch()
    b.forces[2:5] = float("nan")  # graph 1 carries no force labels either
    pe = torch.tensor([[1.5], [2.0], [2.0]], requires_grad=True)
    pf = torch.zeros(6, 3, requires_grad=True)
    loss = EnergyMSELoss(ignore_nonfinite=True) + ForceMSELoss(ignore_nonfinite=True) + ForceL2NormLoss(ignore_nonfinite=True, name="l2")
    out = loss({"energy": pe, "forces": pf}, b)
    out["total_loss"].backward()
    # energy per atom: graphs 0 and 2 -> ((0.5/2)^2 + (1/1)^2) / 2
    assert float(out["EnergyMSELoss[energy]"]) == pytest.approx((0.0625 + 1.0) / 2)
    f = b.forces
    want_f = (f[:2].pow(2).mean() + f[5:].pow(2).mean()) / 2
    assert float(out["ForceMSELoss[forces]"]) == pytest.approx(float(want_f), rel=1e-6)
    want_l2 = (f[:2].norm(dim=-1).mean() + f[5:].norm(dim=-1).mean()) / 2
    assert float(out["l2"]) == pytest.approx(float(want_l2), rel=1e-6)
    assert torch.isfinite(pe.grad).all() and float(pe.grad[1].abs()) == 0.0
    assert torch.isfinite(pf.grad).all() and float(pf.grad[2:5].abs().sum()) == 0.0
    assert loss.per_sample_losses()["ForceMSELoss[forces]"].tolist()[1] == 0.0
    # every label missing: the value is 0, not NaN
    b.energy = torch.full((3,), float("nan"))
    assert float(EnergyMSELoss(ignore_nonfinite=True)({"energy": pe.detach()}, b)) == 0.0
    # without the option a missing label poisons the value (the default stays strict about data)
    assert not torch.isfinite(EnergyMSELoss()({"energy": pe.detach()}, b))


def test_force_loss_reductions_dense_and_padded_agree():
    from nvalchemi_toolkit_b200.training.losses import ForceMSELoss

    b = _mixed_batch()
    g = torch.Generator().manual_seed(0)
    pf = torch.randn(6, 3, generator=g)
    balanced = ForceMSELoss()({"forces": pf}, b)
    d2 = (pf - b.forces) ** 2
    assert float(balanced) == pytest.approx(float((d2[:2].mean() + d2[2:5].mean() + d2[5:].mean()) / 3), rel=1e-6)
    flat = ForceMSELoss(normalize_by_atom_count=False)({"forces": pf}, b)
    assert float(flat) == pytest.approx(float(d2.mean()), rel=1e-6)
    # the same data padded to [B, V_max, 3]; padding rows hold garbage that must not count
    pad_p, pad_t = torch.full((3, 3, 3), 7.0), torch.full((3, 3, 3), -5.0)
    for gi, (lo, hi) in enumerate([(0, 2), (2, 5), (5, 6)]):
        pad_p[gi, : hi - lo], pad_t[gi, : hi - lo] = pf[lo:hi], b.forces[lo:hi]
    for counts in (torch.tensor([2, 3, 1]), torch.tensor([[1, 1, 0], [1, 1, 1], [1, 0, 0]], dtype=torch.bool)):
        pb = _Labels(num_graphs=3, num_nodes_per_graph=counts, forces=pad_t)
        assert float(ForceMSELoss()({"forces": pad_p}, pb)) == pytest.approx(float(balanced), rel=1e-6)
        assert float(ForceMSELoss(normalize_by_atom_count=False)({"forces": pad_p}, pb)) == pytest.approx(float(flat), rel=1e-6)


def test_energy_atom_weighted_reduction_and_dtype_policies():
    from nvalchemi_toolkit_b200.training.losses import ComposedLossFunction, EnergyMSELoss

    b = _mixed_batch()
    b.energy = torch.tensor([1.0, 2.0, 3.0])
    pe = torch.tensor([[2.0], [5.0], [3.5]])
    n = torch.tensor([2.0, 3.0, 1.0])
    per_atom_sq = ((pe[:, 0] - b.energy) / n) ** 2
    assert float(EnergyMSELoss(atom_weighted=True)({"energy": pe}, b)) == pytest.approx(float((n * per_atom_sq).sum() / n.sum()))
    assert float(EnergyMSELoss()({"energy": pe}, b)) == pytest.approx(float(per_atom_sq.mean()))
    with pytest.raises(ValueError, match="per_atom"):
        EnergyMSELoss(per_atom=False, atom_weighted=True)
    with pytest.raises(ValueError, match="shape"):
        EnergyMSELoss()({"energy": pe[:2]}, b)
    b.energy = b.energy.double()
    with pytest.raises(TypeError, match="dtype_policy"):
        EnergyMSELoss(dtype_policy="strict")({"energy": pe}, b)
    strict = EnergyMSELoss(dtype_policy="strict")
    out = ComposedLossFunction([strict], dtype_policy="prediction_to_target")({"energy": pe}, b)
    assert out["total_loss"].dtype == torch.float64 and strict.dtype_policy == "strict"


def test_composed_loss_weight_normalisation_targets_and_supervised_helper():
    from nvalchemi_toolkit_b200.training import (as_composed_loss, assemble_loss_targets, compute_supervised_loss,
                                                 loss_target_keys)
    from nvalchemi_toolkit_b200.training.losses import ComposedLossFunction, EnergyMSELoss, ForceMSELoss, LinearWeight

    e, f = EnergyMSELoss(weight=1.0), ForceMSELoss(weight=LinearWeight(1.0, 3.0, 10))
    loss = ComposedLossFunction([e, f], normalize_weights=True)
    assert loss.weights_at(0) == {e.name: 0.5, f.name: 0.5}
    assert loss.weights_at(10) == {e.name: 0.25, f.name: 0.75}
    with pytest.raises(ValueError, match="sum to zero"):
        ComposedLossFunction([EnergyMSELoss(weight=0.0)], normalize_weights=True).weights_at(0)
    with pytest.raises(ValueError, match="unique"):
        ComposedLossFunction([EnergyMSELoss(), EnergyMSELoss()])
    nested = ComposedLossFunction([ComposedLossFunction([e]), f])
    assert [t.name for t in nested.terms] == [e.name, f.name] and nested.requires_eval_grad
    assert not as_composed_loss(e).requires_eval_grad
    assert loss_target_keys(sum([e, f, EnergyMSELoss(name="again")])) == ("energy", "forces")
    b = _mixed_batch()
    b.energy = torch.tensor([1.0, 2.0, 3.0])
    assert set(assemble_loss_targets(loss, b)) == {"energy", "forces"}
    del b.__dict__["forces"]
    with pytest.raises(KeyError, match="forces"):
        assemble_loss_targets(loss, b)
    assert set(assemble_loss_targets(loss, b, strict=False)) == {"energy"}
    with pytest.raises(KeyError, match="also needs"):
        compute_supervised_loss(lambda batch: {"energy": torch.zeros(3, 1)}, nested, _mixed_batch())
    losses, preds = compute_supervised_loss(lambda batch: {"energy": torch.zeros(3, 1)}, e, b)
    assert set(preds) == {"energy"} and float(losses["total_loss"]) > 0
    round_trip = ComposedLossFunction.from_spec(ComposedLossFunction([EnergyMSELoss(atom_weighted=True, ignore_nonfinite=True),
                                                                      ForceMSELoss(normalize_by_atom_count=False)]).to_spec())
    assert round_trip.terms[0].atom_weighted and round_trip.terms[0].ignore_nonfinite and not round_trip.terms[1].normalize_by_atom_count


def test_runtime_helpers_freeze_and_mode_contexts_and_rank_resolution(monkeypatch):
    from types import SimpleNamespace

    from nvalchemi_toolkit_b200.training import distributed as tdist
    from nvalchemi_toolkit_b200.training import runtime

    models = {"main": torch.nn.Linear(2, 2), "teacher": torch.nn.Linear(2, 2)}
    models["teacher"].bias.requires_grad_(False)  # already frozen by the user: must stay frozen afterwards
    models["teacher"].eval()
    with runtime.freeze_unconfigured_models(models, {"main": object()}):
        assert all(p.requires_grad for p in models["main"].parameters())
        assert not any(p.requires_grad for p in models["teacher"].parameters())
    assert models["teacher"].weight.requires_grad and not models["teacher"].bias.requires_grad
    with runtime.train_configured_models(models, {"main": object()}):
        assert models["main"].training and not models["teacher"].training
        models["teacher"].train()  # whatever happens inside ...
    assert models["main"].training and not models["teacher"].training  # ... the modes of before come back
    try:
        with runtime.freeze_unconfigured_models(models, {}):
            raise KeyError("boom")
    except KeyError:
        pass
    assert models["main"].weight.requires_grad  # restored on the error path too
    moved = runtime.move_to_devices(models, ["cpu"])
    assert set(moved) == {"main", "teacher"} and moved["teacher"].weight.device.type == "cpu"
    with pytest.raises(NotImplementedError, match="DDPHook"):
        runtime.configure_parallelism("fsdp")
    runtime.configure_parallelism("none")
    with pytest.raises(TypeError):
        runtime.validate_training_fn(lambda batch: None)
    runtime.validate_training_fn(lambda model, batch: None)
    # rank resolution: a manager object wins, then the process group, then the launcher's environment
    manager = SimpleNamespace(rank=3, world_size=8, local_rank=1)
    assert (tdist.get_rank(manager), tdist.get_world_size(manager), tdist.get_local_rank(manager)) == (3, 8, 1)
    monkeypatch.setenv("RANK", "5")
    monkeypatch.setenv("WORLD_SIZE", "6")
    monkeypatch.setenv("LOCAL_RANK", "2")
    assert (tdist.get_rank(), tdist.get_world_size(), tdist.get_local_rank()) == (5, 6, 2)
    t = torch.tensor([2.0])
    assert tdist.all_reduce(t, "max") is t and float(t) == 2.0  # no process group: identity
    tdist.barrier()
    tdist.destroy_distributed()
