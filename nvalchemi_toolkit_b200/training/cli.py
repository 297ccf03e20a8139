# SPDX-License-Identifier: Apache-2.0
"""Command line for training jobs: ``python -m nvalchemi_toolkit_b200.training.cli <group> <command>``.

Reference: ``nvalchemi/training/cli.py:165-2229``: click groups ``train`` (``run`` / ``resume``), ``finetune``,
``init`` (write a template job file), ``schema`` (JSON schema of the job file), ``spec`` (``validate`` / ``show``); a job
is a ``TrainingJobSpec`` read from JSON or YAML; a run ends with a report (final losses, learning-rate curve,
warnings).  Classes are named by dotted import paths; nothing is unpickled.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Any

import click
import torch
from pydantic import BaseModel, ConfigDict, Field, model_validator

from nvalchemi_toolkit_b200._serialization import import_from_path


class ComponentSpec(BaseModel):
    """``cls`` (dotted path) called with ``kwargs``; ``checkpoint`` (optional) is passed to ``cls.from_checkpoint``."""

    model_config = ConfigDict(populate_by_name=True)
    cls: str
    kwargs: dict[str, Any] = Field(default_factory=dict)
    checkpoint: str | None = None

    def build(self) -> Any:
        klass = import_from_path(self.cls)
        if self.checkpoint is not None:
            return klass.from_checkpoint(self.checkpoint, **self.kwargs)
        return klass(**self.kwargs)


class DataSpec(BaseModel):
    train: str
    validation: str | None = None
    batch_size: int = 8
    shuffle: bool = True
    drop_last: bool = False
    num_workers: int = 2
    neighbor_cutoff: float | None = None  # build neighbour data per batch when the store has none


class OptimizerSpec(BaseModel):
    cls: str = "torch.optim.Adam"
    kwargs: dict[str, Any] = Field(default_factory=lambda: {"lr": 1e-3})
    scheduler_cls: str | None = None
    scheduler_kwargs: dict[str, Any] = Field(default_factory=dict)
    scheduler_metric: str | None = None
    scheduler_interval: str = "step"


class ValidationSpec(BaseModel):
    every_n_steps: int | None = None
    every_n_epochs: int | None = 1


class ReportingSpec(BaseModel):
    rich: bool = False
    tensorboard_dir: str | None = None
    jsonl: str | None = "metrics.jsonl"
    frequency: int = 1


class FineTuneSpec(BaseModel):
    checkpoint: str
    trainable: list[str] = Field(default_factory=list)
    strict: bool = False


class TrainingJobSpec(BaseModel):
    model: ComponentSpec
    data: DataSpec
    loss: list[dict[str, Any]] = Field(default_factory=lambda: [
        {"cls": "EnergyMSELoss", "weight": 1.0}, {"cls": "ForceMSELoss", "weight": 10.0}])
    #: dtype policy applied to every loss term (``None``: each term's own) and weight normalisation of the composition
    loss_dtype_policy: str | None = None
    normalize_loss_weights: bool = False
    optimizer: OptimizerSpec = Field(default_factory=OptimizerSpec)
    num_epochs: int | None = None
    num_steps: int | None = None
    hooks: list[ComponentSpec] = Field(default_factory=list)
    validation: ValidationSpec | None = None
    reporting: ReportingSpec = Field(default_factory=ReportingSpec)
    finetune: FineTuneSpec | None = None
    output_dir: str = "runs/job"
    checkpoint_every_n_steps: int | None = None
    checkpoint_every_n_epochs: int | None = 1
    devices: list[str] | None = None
    seed: int = 0
    active_outputs: list[str] = Field(default_factory=lambda: ["energy", "forces"])

    @model_validator(mode="after")
    def _one_budget(self) -> "TrainingJobSpec":
        if (self.num_epochs is None) == (self.num_steps is None):
            raise ValueError("give exactly one of num_epochs / num_steps")
        return self

    @classmethod
    def from_file(cls, path: str | Path) -> "TrainingJobSpec":
        path = Path(path)
        text = path.read_text()
        if path.suffix in (".yaml", ".yml"):
            import yaml

            return cls.model_validate(yaml.safe_load(text))
        return cls.model_validate(json.loads(text))

    def to_file(self, path: str | Path) -> None:
        path = Path(path)
        data = self.model_dump(mode="json")
        if path.suffix in (".yaml", ".yml"):
            import yaml

            path.write_text(yaml.safe_dump(data, sort_keys=False))
        else:
            path.write_text(json.dumps(data, indent=2))


MODEL_TEMPLATES: dict[str, dict[str, Any]] = {
    "mace": {"cls": "nvalchemi_toolkit_b200.models.mace.MACEWrapper",
             "kwargs": {"atomic_numbers": [1, 6, 8], "channels": 64, "r_max": 5.0}, "cutoff": 5.0},
    "aimnet2": {"cls": "nvalchemi_toolkit_b200.models.aimnet2.AIMNet2Wrapper", "kwargs": {}, "cutoff": 5.0},
    "demo": {"cls": "nvalchemi_toolkit_b200.models.demo.DemoModelWrapper", "kwargs": {}, "cutoff": None},
    "custom": {"cls": "my_package.my_module.MyModelWrapper", "kwargs": {}, "cutoff": 5.0},
}


def template_spec(workflow: str = "train", model: str = "mace", dataset: str = "data/train.zarr",
                  validation_path: str | None = "data/val.zarr", output_dir: str = "runs/job", lr: float | None = None,
                  num_steps: int | None = None, num_epochs: int | None = None, device: str | None = None,
                  trainable: tuple[str, ...] = (), checkpoint: str | None = None, loss_dtype_policy: str | None = None,
                  validation_every_epochs: int | None = None, validation_every_steps: int | None = None,
                  batch_size: int = 16) -> TrainingJobSpec:
    """A job file to start from (reference ``training/cli.py:1671-2030``: ``init`` per workflow and model family).

    ``workflow="finetune"`` adds the fine-tuning block (checkpoint to start from, patterns of the parameters that stay
    trainable), lowers the default learning rate to the fine-tuning default and drops the scheduler; ``model`` picks the
    wrapper class and its constructor arguments (``custom``: a placeholder import path to edit)."""
    from nvalchemi_toolkit_b200.training.finetune import DEFAULT_FINETUNE_LR

    if workflow not in ("train", "finetune"):
        raise ValueError(f"workflow must be 'train' or 'finetune', got {workflow!r}")
    if model not in MODEL_TEMPLATES:
        raise ValueError(f"model must be one of {sorted(MODEL_TEMPLATES)}, got {model!r}")
    if num_steps is not None and num_epochs is not None:
        raise ValueError("give at most one of num_steps / num_epochs")
    m = MODEL_TEMPLATES[model]
    fine = workflow == "finetune"
    if num_steps is None and num_epochs is None:
        num_epochs = 10
    if validation_path is None:
        validation = None
    elif validation_every_steps is not None:
        validation = ValidationSpec(every_n_steps=validation_every_steps, every_n_epochs=None)
    else:
        validation = ValidationSpec(every_n_epochs=validation_every_epochs or 1)
    optimizer = OptimizerSpec(kwargs={"lr": lr if lr is not None else (DEFAULT_FINETUNE_LR if fine else 1e-3)},
                              scheduler_cls=None if fine else "torch.optim.lr_scheduler.ExponentialLR",
                              scheduler_kwargs={} if fine else {"gamma": 0.999})
    finetune = None
    if fine:
        finetune = FineTuneSpec(checkpoint=checkpoint or "checkpoints/pretrained", trainable=list(trainable) or ["readout"])
    elif trainable or checkpoint:
        raise ValueError("--trainable / --checkpoint belong to the finetune workflow")
    return TrainingJobSpec(
        model=ComponentSpec(cls=m["cls"], kwargs=dict(m["kwargs"])),
        data=DataSpec(train=dataset, validation=validation_path, batch_size=batch_size, neighbor_cutoff=m["cutoff"]),
        num_epochs=num_epochs, num_steps=num_steps, validation=validation, optimizer=optimizer, finetune=finetune,
        output_dir=output_dir, devices=[device] if device else None, loss_dtype_policy=loss_dtype_policy)


# ---- building and running ------------------------------------------------------------------------------------------
class _NeighborTransform:
    """Adds neighbour data to each batch (stores written without edges)."""

    def __init__(self, loader: Any, config: Any) -> None:
        self.loader, self.config = loader, config

    def __len__(self) -> int:
        return len(self.loader)

    def __iter__(self) -> Any:
        from nvalchemi_toolkit_b200 import neighbors as nb

        for batch in self.loader:
            nb.compute_neighbors(batch, config=self.config)
            yield batch

    def __getattr__(self, name: str) -> Any:
        return getattr(self.loader, name)


def _loader(path: str, data: DataSpec, model: Any, shuffle: bool, seed: int) -> Any:
    from nvalchemi_toolkit_b200.data.datapipes import DataLoader, Dataset
    from nvalchemi_toolkit_b200.data.zarr_store import AtomicDataZarrReader

    ds = Dataset(AtomicDataZarrReader(path), num_workers=data.num_workers)
    loader = DataLoader(ds, batch_size=data.batch_size, shuffle=shuffle, drop_last=data.drop_last, seed=seed)
    nc = getattr(getattr(model, "model_config", None), "neighbor_config", None)
    if nc is not None and data.neighbor_cutoff is not None:
        return _NeighborTransform(loader, nc)
    return loader


def build_job(spec: TrainingJobSpec) -> tuple[Any, Any, Any]:
    """``(strategy, train_loader, validation_loader)`` for a job file."""
    from nvalchemi_toolkit_b200.hooks.reporting import JSONLReporter, ReportingOrchestrator, RichReporter, TensorBoardReporter
    from nvalchemi_toolkit_b200.training import ComposedLossFunction, OptimizerConfig, TrainingStrategy, ValidationConfig
    from nvalchemi_toolkit_b200.training.finetune import FineTuningStrategy
    from nvalchemi_toolkit_b200.training.hooks.library import CheckpointHook

    torch.manual_seed(spec.seed)
    model = spec.model.build()
    if hasattr(model, "model_config"):
        model.model_config.active_outputs = set(spec.active_outputs)
    out = Path(spec.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    train = _loader(spec.data.train, spec.data, model, spec.data.shuffle, spec.seed)
    val = _loader(spec.data.validation, spec.data, model, False, spec.seed) if spec.data.validation else None
    hooks: list[Any] = [h.build() for h in spec.hooks]
    hooks.append(CheckpointHook(out / "checkpoints", every_n_steps=spec.checkpoint_every_n_steps,
                                every_n_epochs=spec.checkpoint_every_n_epochs))
    reporters: list[Any] = []
    rep = spec.reporting
    if rep.rich:
        reporters.append(RichReporter(title=f"training {out.name}"))
    if rep.tensorboard_dir:
        reporters.append(TensorBoardReporter(rep.tensorboard_dir))
    if rep.jsonl:
        reporters.append(JSONLReporter(out / rep.jsonl))
    if reporters:
        hooks.append(ReportingOrchestrator(reporters, frequency=rep.frequency, error_policy="warn"))
    vcfg = None
    if spec.validation is not None and val is not None:
        vcfg = ValidationConfig(data=val, every_n_steps=spec.validation.every_n_steps,
                                every_n_epochs=spec.validation.every_n_epochs)
    kw = dict(optimizer_configs=OptimizerConfig(**spec.optimizer.model_dump()), loss_fn=ComposedLossFunction.from_spec(spec.loss, normalize_weights=spec.normalize_loss_weights, dtype_policy=spec.loss_dtype_policy),
              num_epochs=spec.num_epochs, num_steps=spec.num_steps, hooks=hooks, validation_config=vcfg,
              devices=spec.devices)
    if spec.finetune is not None:
        strategy = FineTuningStrategy(model, checkpoint=spec.finetune.checkpoint, trainable=spec.finetune.trainable or None,
                                      strict=spec.finetune.strict, **kw)
    else:
        strategy = TrainingStrategy(model, **kw)
    return strategy, train, val


def final_report(strategy: Any, spec: TrainingJobSpec, console: Any = None) -> dict[str, Any]:
    """Summary table, learning-rate curve and warnings; also written to ``report.json`` in the output directory."""
    from rich.console import Console
    from rich.table import Table

    from nvalchemi_toolkit_b200.hooks.reporting import ReportingOrchestrator, sparkline

    out = Path(spec.output_dir)
    summary: dict[str, Any] = {"steps": strategy.step_count, "epochs": strategy.epoch_count,
                               "losses": {k: float(v) for k, v in (strategy.last_losses or {}).items()
                                          if isinstance(v, torch.Tensor) and v.numel() == 1},
                               "validation": {k: float(v) for k, v in (strategy.last_validation or {}).items()
                                              if isinstance(v, (int, float)) or (isinstance(v, torch.Tensor) and v.numel() == 1)},
                               "warnings": []}
    lr_curve: list[float] = []
    metrics = out / (spec.reporting.jsonl or "metrics.jsonl")
    if metrics.exists():
        for line in metrics.read_text().splitlines():
            row = json.loads(line)
            if "lr/opt0" in row:
                lr_curve.append(row["lr/opt0"])
    for hook in strategy.hooks:
        if isinstance(hook, ReportingOrchestrator):
            summary["warnings"] += [m.text for m in hook.state.messages if m.level in ("warning", "error")]
    if summary["losses"] and any(v != v for v in summary["losses"].values()):
        summary["warnings"].append("a loss term is NaN")
    summary["lr_curve"] = lr_curve[-200:]
    table = Table(title=f"job {out.name}: {summary['steps']} steps, {summary['epochs']} epochs")
    table.add_column("quantity")
    table.add_column("value", justify="right")
    for k, v in summary["losses"].items():
        table.add_row(f"loss/{k}", f"{v:.6g}")
    for k, v in summary["validation"].items():
        table.add_row(f"validation/{k}", f"{v:.6g}")
    if lr_curve:
        table.add_row("learning rate", f"{lr_curve[0]:.3g} → {lr_curve[-1]:.3g}  {sparkline(lr_curve, 40)}")
    for w in summary["warnings"]:
        table.add_row("warning", w)
    (console or Console()).print(table)
    (out / "report.json").write_text(json.dumps(summary, indent=2))
    return summary


def run_job(spec: TrainingJobSpec, resume: bool = False, console: Any = None) -> dict[str, Any]:
    strategy, train, val = build_job(spec)
    out = Path(spec.output_dir)
    spec.to_file(out / "job.json")
    if resume:
        ckpt_dir = out / "checkpoints"
        if not (ckpt_dir / "manifest.json").exists():
            raise click.ClickException(f"nothing to resume from in {ckpt_dir}")
        strategy.load_checkpoint(ckpt_dir)
    strategy.run(train, val)
    return final_report(strategy, spec, console)


# ---- click groups ----------------------------------------------------------------------------------------------------
@click.group()
def main() -> None:
    """Training jobs described by a JSON / YAML file."""


@main.group()
def train() -> None:
    """Run or resume a training job."""


@train.command("run")
@click.argument("job", type=click.Path(exists=True))
@click.option("--output-dir", default=None, help="override the job file's output_dir")
def train_run(job: str, output_dir: str | None) -> None:
    spec = TrainingJobSpec.from_file(job)
    if output_dir:
        spec.output_dir = output_dir
    run_job(spec)


@train.command("resume")
@click.argument("job", type=click.Path(exists=True))
@click.option("--output-dir", default=None)
def train_resume(job: str, output_dir: str | None) -> None:
    spec = TrainingJobSpec.from_file(job)
    if output_dir:
        spec.output_dir = output_dir
    run_job(spec, resume=True)


@main.command("finetune")
@click.argument("job", type=click.Path(exists=True))
@click.option("--checkpoint", default=None, help="weights to start from (overrides finetune.checkpoint)")
@click.option("--trainable", multiple=True, help="parameter-name patterns that stay trainable")
def finetune(job: str, checkpoint: str | None, trainable: tuple[str, ...]) -> None:
    """Run a job as fine-tuning from a checkpoint."""
    spec = TrainingJobSpec.from_file(job)
    base = spec.finetune or (FineTuneSpec(checkpoint=checkpoint) if checkpoint else None)
    if base is None:
        raise click.ClickException("no checkpoint: give --checkpoint or a finetune section")
    if checkpoint:
        base.checkpoint = checkpoint
    if trainable:
        base.trainable = list(trainable)
    spec.finetune = base
    run_job(spec)


def _emit(payload: dict[str, Any], path: str | None, force: bool) -> None:
    """A job / schema document to a file (JSON or YAML by extension) or to the terminal."""
    if path is None:
        click.echo(json.dumps(payload, indent=2))
        return
    target = Path(path)
    if target.exists() and not force:
        raise click.ClickException(f"{path} exists (use --force)")
    target.parent.mkdir(parents=True, exist_ok=True)
    if target.suffix in (".yaml", ".yml"):
        import yaml

        target.write_text(yaml.safe_dump(payload, sort_keys=False))
    else:
        target.write_text(json.dumps(payload, indent=2))
    click.echo(f"wrote {path}")


def _template_options(fn: Any) -> Any:
    for opt in reversed([
        click.option("--workflow", type=click.Choice(["train", "finetune"]), default="train", show_default=True),
        click.option("--model", type=click.Choice(sorted(MODEL_TEMPLATES)), default="mace", show_default=True),
        click.option("--dataset", default="data/train.zarr", show_default=True, help="training store"),
        click.option("--validation-path", default="data/val.zarr", show_default=True, help="'' for none"),
        click.option("--validation-every-epochs", type=int, default=None),
        click.option("--validation-every-steps", type=int, default=None),
        click.option("--output-dir", default="runs/job", show_default=True),
        click.option("--lr", type=float, default=None, help="default: 1e-3 (train), the fine-tuning default (finetune)"),
        click.option("--num-steps", type=int, default=None),
        click.option("--num-epochs", type=int, default=None),
        click.option("--batch-size", type=int, default=16, show_default=True),
        click.option("--device", default=None, help="e.g. cuda:0 (default: chosen at run time)"),
        click.option("--checkpoint", default=None, help="finetune: checkpoint directory to start from"),
        click.option("--trainable", multiple=True, help="finetune: parameter-name patterns that stay trainable"),
        click.option("--loss-dtype-policy", type=click.Choice(["strict", "prediction_to_target", "target_to_prediction"]),
                     default=None),
    ]):
        fn = opt(fn)
    return fn


def _template_from_options(kw: dict[str, Any]) -> TrainingJobSpec:
    kw = dict(kw)
    kw["validation_path"] = kw["validation_path"] or None
    kw["trainable"] = tuple(kw.get("trainable") or ())
    try:
        return template_spec(**kw)
    except ValueError as exc:
        raise click.ClickException(str(exc)) from exc


@main.command("init")
@click.argument("path", type=click.Path(), required=False)
@click.option("--force", is_flag=True)
@_template_options
def init(path: str | None, force: bool, **options: Any) -> None:
    """Write a template job file (JSON or YAML by extension; to the terminal without PATH)."""
    _emit(_template_from_options(options).model_dump(mode="json"), path, force)


@main.group("schema", invoke_without_command=True)
@click.pass_context
def schema(ctx: click.Context) -> None:
    """JSON schema of a job file and templates, for authoring job files offline."""
    if ctx.invoked_subcommand is None:
        click.echo(json.dumps(TrainingJobSpec.model_json_schema(), indent=2))


@schema.command("dump")
@click.option("--out", "output", type=click.Path(), default=None, help="write the schema to this file")
@click.option("--force", is_flag=True)
def schema_dump(output: str | None, force: bool) -> None:
    """The JSON schema of a job file."""
    _emit(TrainingJobSpec.model_json_schema(), output, force)


@schema.command("template")
@click.option("--out", "output", type=click.Path(), default=None, help="write the template to this file")
@click.option("--force", is_flag=True)
@_template_options
def schema_template(output: str | None, force: bool, **options: Any) -> None:
    """A template job for one workflow and model family (same options as ``init``)."""
    _emit(_template_from_options(options).model_dump(mode="json"), output, force)


@main.group()
def spec() -> None:
    """Inspect job files."""


@spec.command("validate")
@click.argument("job", type=click.Path(exists=True))
def spec_validate(job: str) -> None:
    try:
        TrainingJobSpec.from_file(job)
    except Exception as exc:  # noqa: BLE001 - report every validation problem the same way
        raise click.ClickException(f"invalid job file: {exc}") from exc
    click.echo("ok")


@spec.command("show")
@click.argument("job", type=click.Path(exists=True))
def spec_show(job: str) -> None:
    click.echo(json.dumps(TrainingJobSpec.from_file(job).model_dump(mode="json"), indent=2))


# ---- dry-run review of a job file ---------------------------------------------------------------------------------
def job_warnings(job: TrainingJobSpec) -> list[tuple[str, str]]:
    """``(severity, message)`` findings a reviewer would raise before spending GPU hours on the job (reference
    ``training/cli.py`` ``_training_warnings``): paths that do not exist, no validation data, no checkpoints, a plateau
    scheduler without the validation it listens to, force training without forces in the active outputs, a fine-tune
    that trains nothing."""
    out: list[tuple[str, str]] = []
    for label, value in (("data.train", job.data.train), ("data.validation", job.data.validation),
                         ("model.checkpoint", job.model.checkpoint), ("finetune.checkpoint", job.finetune.checkpoint if job.finetune else None)):
        if value is not None and "://" not in str(value) and not Path(value).exists():
            out.append(("error", f"{label}: path '{value}' does not exist"))
    if job.data.validation is None:
        out.append(("warning", "no validation data: over-fitting will go unnoticed and metric-driven schedulers cannot step"))
    elif job.validation is None:
        out.append(("warning", "validation data is given but no validation schedule (validation: {every_n_epochs: 1})"))
    if job.checkpoint_every_n_steps is None and job.checkpoint_every_n_epochs is None and not any(
            "Checkpoint" in h.cls for h in job.hooks):
        out.append(("warning", "no checkpoint cadence and no checkpoint hook: a crash loses the run"))
    o = job.optimizer
    if o.scheduler_cls and "ReduceLROnPlateau" in o.scheduler_cls:
        if o.scheduler_interval != "validation" or job.data.validation is None:
            out.append(("error", "ReduceLROnPlateau steps on a validation metric: set scheduler_interval: validation and give "
                                 "validation data"))
        if not o.scheduler_metric:
            out.append(("warning", "ReduceLROnPlateau without scheduler_metric: defaulting is ambiguous, name the loss key"))
    losses = [str(term.get("cls", "")) for term in job.loss]
    if any("Force" in c for c in losses) and "forces" not in job.active_outputs:
        out.append(("error", "the loss has a force term but 'forces' is not in active_outputs"))
    if any("Stress" in c for c in losses) and "stress" not in job.active_outputs:
        out.append(("error", "the loss has a stress term but 'stress' is not in active_outputs"))
    if job.finetune is not None and not job.finetune.trainable:
        out.append(("info", "fine-tune without a trainable filter: every parameter is trained (full fine-tune)"))
    if job.num_steps is not None and job.checkpoint_every_n_steps and job.checkpoint_every_n_steps > job.num_steps:
        out.append(("warning", "checkpoint_every_n_steps exceeds num_steps: only the final checkpoint will be written"))
    if float(o.kwargs.get("lr", 1e-3)) > 0.1:
        out.append(("warning", f"learning rate {o.kwargs.get('lr')} is unusually large for Adam-family optimisers"))
    return out


def lr_preview(job: TrainingJobSpec, total_steps: int, samples: int = 12) -> list[tuple[int, float]]:
    """Learning rate at ``samples`` points of the run, by stepping the configured scheduler on a dummy parameter (schedulers
    driven by validation metrics stay at the base rate)."""
    import torch

    o = job.optimizer
    p = torch.nn.Parameter(torch.zeros(1))
    opt = import_from_path(o.cls)([p], **o.kwargs)
    sched = None
    if o.scheduler_cls and "ReduceLROnPlateau" not in o.scheduler_cls and o.scheduler_interval == "step":
        sched = import_from_path(o.scheduler_cls)(opt, **o.scheduler_kwargs)
    marks = sorted({int(round(i * max(total_steps - 1, 0) / max(samples - 1, 1))) for i in range(samples)})
    out, step = [], 0
    for target in marks:
        while step < target:
            opt.step()
            if sched is not None:
                sched.step()
            step += 1
        out.append((target, float(opt.param_groups[0]["lr"])))
    return out


def render_report(job: TrainingJobSpec, steps_per_epoch: int | None = None) -> str:
    """Plain-text review of a job: what will run, in which hook order, with which learning-rate curve, and the warnings."""
    lines = ["== job ==", f"model      {job.model.cls}" + (f"  <- {job.model.checkpoint}" if job.model.checkpoint else ""),
             f"data       train={job.data.train}  validation={job.data.validation}  batch_size={job.data.batch_size}",
             f"budget     " + (f"{job.num_epochs} epochs" if job.num_epochs is not None else f"{job.num_steps} steps"),
             f"loss       " + " + ".join(f"{t.get('weight', 1.0)} x {t.get('cls')}" for t in job.loss),
             f"optimizer  {job.optimizer.cls} {job.optimizer.kwargs}" + (
                 f"  scheduler {job.optimizer.scheduler_cls} {job.optimizer.scheduler_kwargs} every {job.optimizer.scheduler_interval}"
                 if job.optimizer.scheduler_cls else ""),
             f"outputs    {job.output_dir}  checkpoints every " + (
                 f"{job.checkpoint_every_n_steps} steps" if job.checkpoint_every_n_steps else f"{job.checkpoint_every_n_epochs} epochs")]
    if job.hooks:
        lines.append("== hooks (registration order) ==")
        for h in job.hooks:
            klass = import_from_path(h.cls)
            stage = getattr(klass, "stage", None)
            lines.append(f"  {h.cls.split('.')[-1]:<28} stage={getattr(stage, 'name', 'several')}  priority={getattr(klass, 'priority', 0)}")
    total = job.num_steps if job.num_steps is not None else (job.num_epochs or 1) * (steps_per_epoch or 100)
    lines.append(f"== learning rate over {total} optimiser steps" + ("" if job.num_steps is not None or steps_per_epoch else
                                                                       " (assuming 100 steps per epoch)") + " ==")
    curve = lr_preview(job, total)
    top = max(v for _, v in curve) or 1.0
    for step, lr in curve:
        lines.append(f"  step {step:>8}  lr {lr:.3e}  " + "#" * max(1, int(round(30 * lr / top))))
    found = job_warnings(job)
    lines.append("== findings ==")
    lines += [f"  [{sev}] {msg}" for sev, msg in found] or ["  none"]
    return "\n".join(lines)


@spec.command("report")
@click.argument("job", type=click.Path(exists=True))
@click.option("--steps-per-epoch", type=int, default=None, help="for the learning-rate preview of epoch-budgeted jobs")
@click.option("--strict", is_flag=True, help="exit with status 1 when a finding has severity 'error'")
def spec_report(job: str, steps_per_epoch: int | None, strict: bool) -> None:
    """Dry-run review of a job file: summary, hook order, learning-rate preview, findings."""
    parsed = TrainingJobSpec.from_file(job)
    click.echo(render_report(parsed, steps_per_epoch))
    if strict and any(sev == "error" for sev, _ in job_warnings(parsed)):
        raise click.ClickException("the job file has findings of severity 'error'")


if __name__ == "__main__":
    sys.exit(main())
