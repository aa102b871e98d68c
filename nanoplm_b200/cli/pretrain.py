"""`nanoplm pretrain {run, from-yaml, get-yaml}` (reference: src/nanoplm/cli/pretrain.py).

`from-yaml` is the main entry: it reads the `model`, `pretraining`, `pure_torch` and `resume`
sections, seeds, builds the model and hands over to the training pipeline. `run` takes the same
settings as options (the reference's `run` cannot be invoked because of mismatched option names,
cli/pretrain.py:89-93 vs :351; here it works). `get-yaml` writes the template.
"""
from __future__ import annotations

import random
from pathlib import Path

import click

from nanoplm_b200.config import (ConfigError, ModelConfig, PretrainingConfig, PureTorchConfig, ResumeConfig,
                                 load_model_config, load_pretrain_config, load_resume_config, read_yaml,
                                 resolve_pure_torch_config)
from nanoplm_b200.config.templates import PRETRAIN_YAML
from nanoplm_b200.utils.logging import logger


def set_seed_for_init(seed: int) -> None:
    import numpy as np
    import torch
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def _launch(model_cfg: ModelConfig, cfg: PretrainingConfig, pt: PureTorchConfig, resume: ResumeConfig):
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.runtime.pretrain import run_pretraining
    set_seed_for_init(cfg.seed)
    model = ProtEncoderMLM(model_cfg, ProtTokenizer())
    logger.info(f"Model parameters: {model.num_parameters():,}")
    return run_pretraining(model, cfg, pt, resume)


@click.group(help="Group of commands for model pretraining.")
def pretrain() -> None:
    pass


@pretrain.command("from-yaml", help="Run pretraining from a YAML configuration file.")
@click.argument("config", default="pretrain.yaml", type=click.Path(dir_okay=False, path_type=Path))
def from_yaml(config: Path) -> None:
    path = config if config.is_absolute() else Path.cwd() / config
    if not path.exists():
        raise click.ClickException(f"Config file not found: {path}")
    try:
        raw = read_yaml(path)
        pure_enabled, pt = resolve_pure_torch_config(raw)
        cfg = load_pretrain_config(raw.get("pretraining"))
        model_cfg = load_model_config(raw.get("model"))
        resume = load_resume_config(raw.get("resume"))
    except (ConfigError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    if not pure_enabled:
        pt = _hf_trainer_recipe(cfg, pt)
    _launch(model_cfg, cfg, pt, resume)


def _hf_trainer_recipe(cfg, pt: PureTorchConfig) -> PureTorchConfig:
    """With the pure-torch pipeline switched off the reference runs its HF-Trainer pipeline
    (src/nanoplm/pretraining/pipeline.py:107-295): padded batches from ProtDataCollatorForLM,
    checkpoints with model.safetensors and trainer_state.json. The same recipe on the native
    pipeline: no packing, and every checkpoint also carries the two HF files (the native files stay,
    so either pipeline can resume)."""
    import dataclasses
    cfg.hf_checkpoint_files = True
    logger.info("pure-torch is off: running the reference's HF-Trainer recipe on the native pipeline "
                "(padded batches, checkpoints also carry model.safetensors and trainer_state.json).")
    return dataclasses.replace(pt, use_packing=False)


@pretrain.command("supervise", help="Run `from-yaml` as N supervised ranks: when a rank fails or stalls, end the "
                                    "others and restart from the latest complete checkpoint.")
@click.argument("config", default="pretrain.yaml", type=click.Path(dir_okay=False, path_type=Path))
@click.option("--nproc", type=int, default=1, show_default=True, help="Ranks to start (one per GPU).")
@click.option("--max-restarts", type=int, default=3, show_default=True)
@click.option("--stall-seconds", type=float, default=0.0,
              help="With pretraining.heartbeat_seconds set: restart when a rank's step stops advancing this long.")
@click.option("--grace-seconds", type=float, default=10.0, show_default=True,
              help="Time between SIGTERM and SIGKILL for the ranks of a failed attempt.")
@click.option("--log-dir", type=click.Path(path_type=Path), default=None,
              help="Write every rank's output to <log-dir>/attempt-K-rank-R.log instead of the terminal.")
def supervise(config: Path, nproc: int, max_restarts: int, stall_seconds: float, grace_seconds: float,
              log_dir: Path | None) -> None:
    from nanoplm_b200.runtime.supervisor import Supervisor
    try:
        sup = Supervisor(config if config.is_absolute() else Path.cwd() / config, nproc, max_restarts,
                         stall_seconds, grace_seconds, log_dir=log_dir)
    except (FileNotFoundError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    code = sup.run()
    click.echo(f"attempts: {len(sup.attempts)}, restarts: {sup.restarts}, run directory: {sup.run_dir}")
    if code != 0:
        raise click.ClickException(f"job did not finish within {max_restarts} restart(s): {sup.attempts[-1].reason}")


@pretrain.command("get-yaml", help="Write a pretraining YAML template.")
@click.argument("output", required=False, type=click.Path(path_type=Path))
@click.option("--force", is_flag=True, help="Overwrite an existing file.")
def get_yaml(output: Path | None, force: bool) -> None:
    target = Path.cwd() / "pretrain.yaml" if output is None else output
    if target.is_dir() or (output is not None and not target.suffix):
        target = target / "pretrain.yaml"
    if target.exists() and not force:
        raise click.ClickException(f"File already exists: {target}. Use --force to overwrite.")
    target.parent.mkdir(parents=True, exist_ok=True)
    target.write_text(PRETRAIN_YAML, encoding="utf-8")
    click.echo(f"Template written to: {target}")


def _opt(name, **kw):
    return click.option(f"--{name.replace('_', '-')}", name, **kw)


@pretrain.command("run", help="Run pretraining with settings given as options.")
@_opt("dataset_dir", required=True, type=str)
@_opt("ckp_dir", default="output/pretraining", type=str)
@_opt("micro_batch_size", default=32, type=int)
@_opt("global_batch_size", default=2 ** 20, type=int)
@_opt("num_epochs", default=10, type=int)
@click.option("--warmup-ratio", "--adam-warmup-ratio", "warmup_ratio", default=0.05, type=float,
              help="Warm-up share of the optimizer steps (a value >= 1 is a step count).")
@_opt("optimizer", default="adamw", type=click.Choice(["adamw", "stable_adamw", "muon", "normuon"]))
@_opt("adam_beta1", default=0.9, type=float)
@_opt("adam_beta2", default=0.999, type=float)
@_opt("adam_epsilon", default=1e-8, type=float)
@_opt("adam_learning_rate", default=1e-3, type=float)
@_opt("adam_weight_decay", default=0.0, type=float)
@_opt("muon_learning_rate", default=2e-2, type=float)
@_opt("muon_weight_decay", default=0.1, type=float)
@_opt("muon_momentum", default=0.95, type=float)
@_opt("muon_eps", default=1e-7, type=float)
@click.option("--muon-nesterov/--no-muon-nesterov", "muon_nesterov", default=True)
@click.option("--muon-cautious-weight-decay/--no-muon-cautious-weight-decay", "muon_cautious_weight_decay", default=True)
@click.option("--muon-use-polar-express/--no-muon-use-polar-express", "muon_use_polar_express", default=False)
@_opt("mlm_probability", default=0.3, type=float)
@_opt("mask_replace_prob", default=0.8, type=float)
@_opt("random_token_prob", default=0.1, type=float)
@_opt("keep_probability", default=0.1, type=float)
@_opt("logging_steps", default=10, type=int)
@_opt("eval_steps", default=50, type=int)
@_opt("save_steps", default=100, type=int)
@_opt("seed", default=42, type=int)
@_opt("num_workers", default="auto", type=str)
@_opt("prefetch_factor", default=2, type=int)
@click.option("--bf16/--no-bf16", default=True)
@click.option("--tf32/--no-tf32", default=True)
@click.option("--multi-gpu/--no-multi-gpu", "multi_gpu", default=False)
@_opt("world_size", default="1", type=str)
@_opt("project_name", default="nanoplm-pretraining", type=str)
@click.option("--fp8/--no-fp8", default=False)
@click.option("--fused-comm/--no-fused-comm", "fused_comm", default=True)
@_opt("hidden_size", default=1024, type=int)
@_opt("intermediate_size", default=2048, type=int)
@_opt("num_hidden_layers", default=16, type=int)
@_opt("num_attention_heads", default=16, type=int)
@_opt("vocab_size", default=32, type=int)
@_opt("mlp_activation", default="swiglu", type=str)
@_opt("mlp_dropout", default=0.0, type=float)
@click.option("--mlp-bias/--no-mlp-bias", "mlp_bias", default=False)
@click.option("--attention-bias/--no-attention-bias", "attention_bias", default=False)
@_opt("attention_dropout", default=0.0, type=float)
@_opt("classifier_activation", default="gelu", type=str)
@_opt("max_position_embeddings", default=1024, type=int)
@click.option("--pure-torch/--no-pure-torch", "pure_torch", default=True,
              help="--no-pure-torch runs the HF-Trainer recipe (padded batches, HF files in the checkpoints).")
@click.option("--compile/--no-compile", "use_compile", default=True,
              help="Accepted for compatibility: there is no compiler step here.")
@click.option("--use-packing/--no-packing", "use_packing", default=False)
@click.option("--no-use-packing", "use_packing", flag_value=False, hidden=True)
@_opt("target_packed_rows", default=None, type=int)
@_opt("resume_from", default=None, type=str, help="checkpoint-N directory to resume from")
@_opt("extra_epochs", default=None, type=int)
def run(**kw) -> None:
    model_keys = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                  "mlp_activation", "mlp_dropout", "mlp_bias", "attention_bias", "attention_dropout",
                  "classifier_activation", "max_position_embeddings")
    try:
        model_cfg = ModelConfig(**{k: kw.pop(k) for k in model_keys})
        pure_enabled = kw.pop("pure_torch")
        pt = PureTorchConfig(use_compile=kw.pop("use_compile"), use_packing=kw.pop("use_packing"),
                             target_packed_rows=kw.pop("target_packed_rows"))
        resume_from, extra = kw.pop("resume_from"), kw.pop("extra_epochs")
        resume = load_resume_config({"is_resume": bool(resume_from), "checkpoint_dir": resume_from or "",
                                     "extra_epochs": extra})
        ws = kw["world_size"]
        kw["world_size"] = ws if ws == "auto" else int(ws)
        nw = kw["num_workers"]
        kw["num_workers"] = nw if nw == "auto" else int(nw)
        cfg = load_pretrain_config(kw)
    except (ConfigError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    if not pure_enabled:
        pt = _hf_trainer_recipe(cfg, pt)
    _launch(model_cfg, cfg, pt, resume)
