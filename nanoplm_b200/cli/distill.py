"""`nanoplm distill {run, from-yaml, get-yaml}` (reference: src/nanoplm/cli/distill.py)."""
from __future__ import annotations

import json
from pathlib import Path

import click

from nanoplm_b200.config import (ConfigError, load_distill_config, load_resume_config, load_student_config,
                                 read_yaml)
from nanoplm_b200.config.templates import DISTILL_YAML


@click.group(help="Group of commands for embedding distillation.")
def distill() -> None:
    pass


def _launch(model_cfg, cfg, resume):
    from nanoplm_b200.runtime.distill import run_distillation
    return run_distillation(model_cfg, cfg, resume)


@distill.command("from-yaml", help="Run distillation from a YAML configuration file.")
@click.argument("config", default="distill.yaml", type=click.Path(dir_okay=False, path_type=Path))
def from_yaml(config: Path) -> None:
    path = config if config.is_absolute() else Path.cwd() / config
    if not path.exists():
        raise click.ClickException(f"Config file not found: {path}")
    try:
        raw = read_yaml(path)
        if "model" not in raw or "distillation" not in raw:
            raise ConfigError("distill.yaml needs a 'model' and a 'distillation' section")
        model_cfg = load_student_config(raw.get("model"))
        cfg = load_distill_config(raw.get("distillation"))
        resume = load_resume_config(raw.get("resume"))
    except (ConfigError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    _launch(model_cfg, cfg, resume)


@distill.command("supervise", help="Run `from-yaml` as N supervised ranks: when a rank fails, end the others and "
                                   "restart from the latest complete checkpoint.")
@click.argument("config", default="distill.yaml", type=click.Path(dir_okay=False, path_type=Path))
@click.option("--nproc", type=int, default=1, show_default=True, help="Ranks to start (one per GPU).")
@click.option("--max-restarts", type=int, default=3, show_default=True)
@click.option("--stall-seconds", type=float, default=0.0,
              help="With distillation.heartbeat_seconds set: restart when a rank's step stops advancing this long.")
@click.option("--grace-seconds", type=float, default=10.0, show_default=True)
@click.option("--log-dir", type=click.Path(path_type=Path), default=None)
def supervise(config: Path, nproc: int, max_restarts: int, stall_seconds: float, grace_seconds: float, log_dir) -> None:
    from nanoplm_b200.runtime.supervisor import Supervisor
    try:
        sup = Supervisor(config if config.is_absolute() else Path.cwd() / config, nproc, max_restarts,
                         stall_seconds=stall_seconds, grace_seconds=grace_seconds, log_dir=log_dir,
                         section="distillation")
    except (FileNotFoundError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    code = sup.run()
    click.echo(f"attempts: {len(sup.attempts)}, restarts: {sup.restarts}, run directory: {sup.run_dir}")
    if code != 0:
        raise click.ClickException(f"job did not finish within {max_restarts} restart(s): {sup.attempts[-1].reason}")


@distill.command("get-yaml", help="Write a distillation YAML template.")
@click.argument("output", required=False, type=click.Path(path_type=Path))
@click.option("--force", is_flag=True)
def get_yaml(output, force) -> None:
    target = Path.cwd() / "distill.yaml" if output is None else Path(output)
    if target.is_dir() or (output is not None and not target.suffix):
        target = target / "distill.yaml"
    if target.exists() and not force:
        raise click.ClickException(f"File already exists: {target}. Use --force to overwrite.")
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(DISTILL_YAML, encoding="utf-8")
    click.echo(f"Template written to: {target}")


def _o(name, **kw):
    return click.option(f"--{name.replace('_', '-')}", name, **kw)


@distill.command("run", help="Run distillation with settings given as options.")
@_o("dataset_dir", default=None, type=str)
@_o("ckp_dir", default="output/distillation", type=str)
@_o("num_epochs", default=10, type=int)
@_o("batch_size", default=64, type=int)
@_o("learning_rate", default=1e-3, type=float)
@_o("gradient_accumulation_steps", default=1, type=int)
@_o("warmup_ratio", default=0.05, type=float)
@_o("lr_scheduler", default="cosine", type=click.Choice(["cosine", "linear", "polynomial", "constant"]))
@_o("lr_scheduler_kwargs", default=None, type=str, help="JSON object with scheduler arguments")
@_o("max_open_files", default=5, type=int)
@_o("chunk_size", default=32, type=int)
@_o("prefetch_batches", default=2, type=int)
@click.option("--use-threading/--no-threading", "use_threading", default=True)
@click.option("--no-use-threading", "use_threading", flag_value=False, hidden=True)
@_o("num_workers", default=8, type=int)
@_o("project_name", default="nanoplm-distillation", type=str)
@_o("logging_steps", default=10, type=int)
@_o("eval_steps", default=50, type=int)
@_o("save_steps", default=100, type=int)
@click.option("--bf16/--no-bf16", default=True)
@click.option("--tf32/--no-tf32", default=True)
@click.option("--multi-gpu/--no-multi-gpu", "multi_gpu", default=False)
@_o("world_size", default="1", type=str)
@_o("seed", default=42, type=int)
@click.option("--teacher-random-init", is_flag=True)
@_o("hidden_size", default=512, type=int)
@_o("intermediate_size", default=1024, type=int)
@_o("num_hidden_layers", default=6, type=int)
@_o("num_attention_heads", default=8, type=int)
@_o("mlp_activation", default="swiglu", type=str)
@_o("mlp_dropout", default=0.0, type=float)
@click.option("--mlp-bias/--no-mlp-bias", "mlp_bias", default=False)
@click.option("--attention-bias/--no-attention-bias", "attention_bias", default=False)
@_o("attention_dropout", default=0.0, type=float)
@_o("classifier_activation", default="gelu", type=str)
@click.option("--projection-layer/--no-projection-layer", "projection_layer", default=True)
@_o("resume_from", default=None, type=str, help="checkpoint-N directory; dataset_dir may be omitted then")
@_o("extra_epochs", default=0, type=int)
def run(**kw) -> None:
    model_keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "mlp_activation",
                  "mlp_dropout", "mlp_bias", "attention_bias", "attention_dropout", "classifier_activation",
                  "projection_layer")
    try:
        model_cfg = load_student_config({k: kw.pop(k) for k in model_keys})
        resume_from, extra = kw.pop("resume_from"), kw.pop("extra_epochs")
        explicit_paths = False
        if resume_from and not kw.get("dataset_dir"):
            # recover the dataset location from the run's training_config.json: the dataset directory
            # when the file was written here, else the explicit paths the reference stores
            # (cli/distill.py:303-337, 406-425)
            if not Path(resume_from).exists():
                raise ConfigError(f"Resume checkpoint directory does not exist: {resume_from}")
            tc = Path(resume_from).parent / "training_config.json"
            if not tc.exists():
                raise ConfigError(f"Cannot resume without --dataset-dir: training_config.json not found in "
                                  f"{tc.parent}\nPlease provide --dataset-dir explicitly.")
            saved = json.loads(tc.read_text())
            kw["dataset_dir"] = (saved.get("distillation") or {}).get("dataset_dir")
            if not kw["dataset_dir"]:
                explicit_paths = True
                for k in ("train_fasta", "val_fasta", "train_h5_prefix", "val_h5_prefix", "max_seq_len",
                          "max_seqs_num", "val_ratio", "on_the_fly", "sharded", "train_sequences", "val_sequences"):
                    v = saved.get(k)
                    kw[k] = None if v in (None, "None", "null") else v
        if kw.get("lr_scheduler_kwargs"):
            kw["lr_scheduler_kwargs"] = json.loads(kw["lr_scheduler_kwargs"])
        else:
            kw.pop("lr_scheduler_kwargs")
        ws = kw["world_size"]
        kw["world_size"] = ws if ws == "auto" else int(ws)
        cfg = load_distill_config(kw, require_dataset_dir=not explicit_paths)
        resume = load_resume_config({"is_resume": bool(resume_from), "checkpoint_dir": resume_from or "",
                                     "extra_epochs": extra})
    except (ConfigError, ValueError, json.JSONDecodeError) as exc:
        raise click.ClickException(str(exc)) from exc
    _launch(model_cfg, cfg, resume)
