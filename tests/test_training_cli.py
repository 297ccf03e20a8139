# SPDX-License-Identifier: Apache-2.0
"""Training CLI: job files, init/schema/spec commands, run + resume + fine-tune on a small Zarr data set."""
import json

import pytest
import torch
from click.testing import CliRunner

from nvalchemi_toolkit_b200 import Batch
from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrWriter
from nvalchemi_toolkit_b200.training import cli
from tests.test_training import _dataset


def _store(path, n, seed):
    AtomicDataZarrWriter(path).append(Batch.from_data_list(_dataset(n, seed)))


def _job(tmp_path, **kw):
    _store(tmp_path / "train.zarr", 12, 0)
    _store(tmp_path / "val.zarr", 4, 1)
    spec = cli.TrainingJobSpec(
        model=cli.ComponentSpec(cls="nvalchemi_toolkit_b200.models.demo.DemoModelWrapper", kwargs={"hidden_dim": 16}),
        data=cli.DataSpec(train=str(tmp_path / "train.zarr"), validation=str(tmp_path / "val.zarr"), batch_size=4, shuffle=False),
        output_dir=str(tmp_path / "run"), devices=["cpu"], validation=cli.ValidationSpec(every_n_epochs=1),
        optimizer=cli.OptimizerSpec(kwargs={"lr": 1e-2}, scheduler_cls="torch.optim.lr_scheduler.ExponentialLR",
                                    scheduler_kwargs={"gamma": 0.9}), **kw)
    path = tmp_path / "job.yaml"
    spec.to_file(path)
    return path


def test_init_schema_and_spec_commands(tmp_path):
    r = CliRunner()
    out = r.invoke(cli.main, ["init", str(tmp_path / "t.json")])
    assert out.exit_code == 0 and json.loads((tmp_path / "t.json").read_text())["model"]["cls"].endswith("MACEWrapper")
    assert r.invoke(cli.main, ["init", str(tmp_path / "t.json")]).exit_code != 0  # refuses to overwrite
    assert r.invoke(cli.main, ["spec", "validate", str(tmp_path / "t.json")]).output.strip() == "ok"
    schema = json.loads(r.invoke(cli.main, ["schema"]).output)
    assert "num_epochs" in schema["properties"] and "model" in schema["required"]
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"model": {"cls": "x.Y"}, "data": {"train": "a"}, "num_epochs": 1, "num_steps": 5}))
    res = r.invoke(cli.main, ["spec", "validate", str(bad)])
    assert res.exit_code != 0 and "exactly one" in res.output
    shown = json.loads(r.invoke(cli.main, ["spec", "show", str(tmp_path / "t.json")]).output)
    assert shown["data"]["neighbor_cutoff"] == 5.0


def test_run_resume_and_finetune(tmp_path):
    job = _job(tmp_path, num_epochs=2)
    r = CliRunner()
    res = r.invoke(cli.main, ["train", "run", str(job)])
    assert res.exit_code == 0, res.output
    run = tmp_path / "run"
    report = json.loads((run / "report.json").read_text())
    assert report["steps"] == 6 and report["epochs"] == 2 and "total_loss" in report["losses"]
    assert len(report["lr_curve"]) == 6 and report["lr_curve"][-1] < report["lr_curve"][0]
    assert (run / "checkpoints" / "manifest.json").exists() and (run / "job.json").exists()
    rows = [json.loads(l) for l in (run / "metrics.jsonl").read_text().splitlines()]
    assert rows[-1]["loss/total"] < rows[0]["loss/total"]
    # resume with a larger budget continues from the stored counters
    spec = cli.TrainingJobSpec.from_file(job)
    spec.num_epochs = 3
    spec.to_file(job)
    res = r.invoke(cli.main, ["train", "resume", str(job)])
    assert res.exit_code == 0, res.output
    assert json.loads((run / "report.json").read_text())["steps"] == 9
    # fine-tune only the projection head from the exported weights
    from nvalchemi_toolkit_b200.models.demo import DemoModelWrapper

    w = DemoModelWrapper(hidden_dim=16)
    torch.save(w.model.state_dict(), tmp_path / "w.pt")
    spec.output_dir, spec.num_epochs = str(tmp_path / "ft"), 1
    spec.to_file(job)
    res = r.invoke(cli.main, ["finetune", str(job), "--checkpoint", str(tmp_path / "w.pt"), "--trainable", "projection"])
    assert res.exit_code == 0, res.output
    assert json.loads((tmp_path / "ft" / "report.json").read_text())["steps"] == 3
    assert r.invoke(cli.main, ["train", "resume", str(job), "--output-dir", str(tmp_path / "nothing")]).exit_code != 0


def test_spec_report_previews_the_schedule_and_lists_findings(tmp_path):
    path = _job(tmp_path, num_steps=50, hooks=[cli.ComponentSpec(cls="nvalchemi_toolkit_b200.training.hooks.library.GradientClipHook",
                                                                  kwargs={"max_norm": 1.0})])
    r = CliRunner()
    out = r.invoke(cli.main, ["spec", "report", str(path)])
    assert out.exit_code == 0, out.output
    text = out.output
    assert "GradientClipHook" in text and "learning rate over 50 optimiser steps" in text and "none" in text.split("== findings ==")[1]
    job = cli.TrainingJobSpec.from_file(path)
    curve = cli.lr_preview(job, 50, samples=3)
    assert curve[0] == (0, 1e-2) and abs(curve[-1][1] - 1e-2 * 0.9 ** 49) < 1e-12
    bad = job.model_copy(update={"data": job.data.model_copy(update={"train": str(tmp_path / "missing.zarr"), "validation": None}),
                                 "active_outputs": ["energy"], "checkpoint_every_n_epochs": None,
                                 "optimizer": cli.OptimizerSpec(cls="torch.optim.Adam", kwargs={"lr": 0.5},
                                                                scheduler_cls="torch.optim.lr_scheduler.ReduceLROnPlateau")})
    found = cli.job_warnings(bad)
    text = " | ".join(m for _, m in found)
    assert "does not exist" in text and "no validation data" in text and "no checkpoint cadence" in text
    assert "ReduceLROnPlateau steps on a validation metric" in text and "force term" in text and "unusually large" in text
    bad.to_file(tmp_path / "bad.yaml")
    assert r.invoke(cli.main, ["spec", "report", str(tmp_path / "bad.yaml"), "--strict"]).exit_code != 0


def test_init_templates_per_workflow_and_schema_subcommands(tmp_path):
    r = CliRunner()
    out = r.invoke(cli.main, ["init", "--workflow", "finetune", "--model", "aimnet2", "--trainable", "readout", "--trainable",
                              "embed.*", "--num-steps", "500", "--checkpoint", "ckpt/base", "--validation-path", "",
                              "--loss-dtype-policy", "prediction_to_target"])
    assert out.exit_code == 0, out.output
    job = cli.TrainingJobSpec.model_validate(json.loads(out.output))  # printed to the terminal, and a valid job
    assert job.finetune.checkpoint == "ckpt/base" and job.finetune.trainable == ["readout", "embed.*"]
    assert job.num_steps == 500 and job.num_epochs is None and job.validation is None and job.data.validation is None
    assert job.optimizer.kwargs["lr"] == pytest.approx(1e-4) and job.optimizer.scheduler_cls is None
    assert job.model.cls.endswith("AIMNet2Wrapper") and job.loss_dtype_policy == "prediction_to_target"
    # options of the other workflow are refused, as are two budgets
    assert r.invoke(cli.main, ["init", "--trainable", "readout"]).exit_code != 0
    assert r.invoke(cli.main, ["init", "--num-steps", "5", "--num-epochs", "2"]).exit_code != 0
    # YAML by extension; validation cadence in steps
    path = tmp_path / "sub" / "job.yaml"
    out = r.invoke(cli.main, ["init", str(path), "--model", "demo", "--validation-every-steps", "50", "--device", "cpu"])
    assert out.exit_code == 0 and path.exists()
    job = cli.TrainingJobSpec.from_file(path)
    assert job.validation.every_n_steps == 50 and job.validation.every_n_epochs is None and job.devices == ["cpu"]
    assert job.data.neighbor_cutoff is None  # the demo model needs no neighbour list
    # schema group: bare call and `dump` agree; `template` takes the same options as `init`
    bare = json.loads(r.invoke(cli.main, ["schema"]).output)
    dumped = tmp_path / "schema.json"
    assert r.invoke(cli.main, ["schema", "dump", "--out", str(dumped)]).exit_code == 0
    assert json.loads(dumped.read_text()) == bare and "loss_dtype_policy" in bare["properties"]
    templ = r.invoke(cli.main, ["schema", "template", "--workflow", "finetune", "--model", "mace"])
    assert json.loads(templ.output)["finetune"]["trainable"] == ["readout"]


def test_job_loss_options_reach_the_composed_loss(tmp_path):
    job = cli.template_spec(model="demo", dataset=str(tmp_path / "none.zarr"), validation_path=None, num_steps=1,
                            loss_dtype_policy="target_to_prediction")
    job.normalize_loss_weights = True
    from nvalchemi_toolkit_b200.training import ComposedLossFunction

    loss = ComposedLossFunction.from_spec(job.loss, normalize_weights=job.normalize_loss_weights, dtype_policy=job.loss_dtype_policy)
    w = loss.weights_at(0)
    assert sum(w.values()) == pytest.approx(1.0) and loss.dtype_policy == "target_to_prediction"
