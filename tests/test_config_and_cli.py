"""YAML loaders, templates and the CLI end to end on CPU (data from-yaml with the built-in stage
runner -> pretrain from-yaml -> resume; distill from-yaml with a tiny random-init teacher)."""
import json
import os
from pathlib import Path

import pytest
import yaml
from click.testing import CliRunner

from nanoplm_b200.cli import cli
from nanoplm_b200.config import (ConfigError, load_model_config, load_pretrain_config, load_resume_config,
                                 resolve_pure_torch_config)
from nanoplm_b200.config.templates import DISTILL_YAML, PARAMS_YAML, PRETRAIN_YAML
from nanoplm_b200.data.synthetic import write_synthetic_fasta


def test_templates_load_with_the_strict_loaders():
    raw = yaml.safe_load(PRETRAIN_YAML)
    m = load_model_config(raw["model"])
    assert (m.hidden_size, m.num_hidden_layers, m.vocab_size) == (1024, 16, 32)
    p = load_pretrain_config(raw["pretraining"])
    assert p.adam_learning_rate == 1e-3 and p.global_batch_size == 2 ** 20 and p.mlm_probability == 0.3
    enabled, pt = resolve_pure_torch_config(raw)
    assert enabled and pt.use_packing and pt.target_packed_rows is None
    assert set(yaml.safe_load(PARAMS_YAML)) == {"data_params", "pretrain_config", "distillation_config", "data_dirs"}
    assert set(yaml.safe_load(DISTILL_YAML)) == {"model", "distillation", "resume"}


def test_loader_rules():
    base = yaml.safe_load(PRETRAIN_YAML)
    model = dict(base["model"])
    model.pop("vocab_size")
    with pytest.raises(ConfigError, match="Missing required model configuration keys: vocab_size"):
        load_model_config(model)
    with pytest.raises(ConfigError, match="Unexpected model configuration keys: bogus"):
        load_model_config({**base["model"], "bogus": 1})
    ok = load_model_config({**base["model"], "conv_kernel_size": 7, "mhc_streams": 4,
                            "moe": {"num_experts": 8, "top_k": 2}})
    assert ok.conv_kernel_size == 7 and ok.moe.enabled and ok.is_moe_layer(1) and not ok.is_moe_layer(0)
    pre = dict(base["pretraining"])
    with pytest.raises(ConfigError, match="gradient_accumulation_steps is inferred"):
        load_pretrain_config({**pre, "gradient_accumulation_steps": 4})
    with pytest.raises(ConfigError, match="dataset_dir is required"):
        load_pretrain_config({k: v for k, v in pre.items() if k != "dataset_dir"})
    with pytest.raises(ConfigError, match="Unexpected training configuration keys: nope"):
        load_pretrain_config({**pre, "nope": 1})
    legacy = {k: v for k, v in pre.items() if k not in ("adam_learning_rate", "adam_weight_decay")}
    cfg = load_pretrain_config({**legacy, "learning_rate": "3e-4", "weight_decay": "0.01", "bf16": "false"})
    assert cfg.adam_learning_rate == 3e-4 and cfg.adam_weight_decay == 0.01 and cfg.bf16 is False
    with pytest.raises(ConfigError, match="Invalid adam_beta1"):
        load_pretrain_config({**pre, "adam_beta1": "abc"})
    extra = load_pretrain_config({**pre, "deterministic_attention": True, "shard_params": True, "balance_ranks": False})
    assert extra.deterministic_attention is True and extra.shard_params is True and extra.balance_ranks is False
    assert load_pretrain_config(pre).deterministic_attention is False
    assert load_resume_config(None).is_resume is False
    with pytest.raises(ConfigError, match="does not exist"):
        load_resume_config({"is_resume": True, "checkpoint_dir": "/nonexistent/ckpt"})
    with pytest.raises(ConfigError, match="missing"):
        load_resume_config({"is_resume": True})


def _write_params(tmp: Path, mode: str, on_the_fly=False):
    params = yaml.safe_load(PARAMS_YAML)
    params["data_params"].update(pipeline_mode=mode, seqs_num=60, min_seq_len=10, max_seq_len=64, val_ratio=0.2)
    params["pretrain_config"].update(output_dir="out/shards", samples_per_shard=20, max_workers=1)
    params["distillation_config"].update(output_dir="out/kd", on_the_fly=on_the_fly)
    params["data_dirs"].update(url="unused", compressed_fasta="raw/x.fasta.gz", extracted_fasta="raw/x.fasta",
                               shuffled_fasta="raw/x_shuf.fasta", filtered_fasta="raw/x_filt.fasta",
                               splitted_fasta_dir="raw/split")
    (tmp / "params.yaml").write_text(yaml.safe_dump(params))
    write_synthetic_fasta(tmp / "raw" / "x.fasta", 120, 5, 80, seed=11)


def test_cli_data_pretrain_resume_cycle(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    runner = CliRunner()
    r = runner.invoke(cli, ["data", "get-yaml", str(tmp_path)])
    assert r.exit_code == 0 and (tmp_path / "dvc.yaml").exists()
    assert runner.invoke(cli, ["data", "get-yaml", str(tmp_path)]).exit_code != 0       # no overwrite
    _write_params(tmp_path, "pretrain")
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "builtin"])
    assert r.exit_code == 0, r.output
    manifest = yaml.safe_load((tmp_path / "out" / "shards" / ".data_manifest").read_text())
    assert manifest["pipeline_mode"] == "pretrain" and manifest["train_sequences"] == 48 and manifest["val_sequences"] == 12

    r = runner.invoke(cli, ["pretrain", "get-yaml", "pretrain.yaml"])
    assert r.exit_code == 0
    cfg = yaml.safe_load((tmp_path / "pretrain.yaml").read_text())
    cfg["model"].update(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                        max_position_embeddings=128)
    cfg["pretraining"].update(dataset_dir="out/shards", ckp_dir="ckpt", micro_batch_size=8, global_batch_size=8 * 64,
                              num_epochs=2, logging_steps=1, eval_steps=3, save_steps=3, num_workers=0, bf16=False)
    cfg["pure_torch"].update(use_packing=True, target_packed_rows=5)
    (tmp_path / "pretrain.yaml").write_text(yaml.safe_dump(cfg))
    r = runner.invoke(cli, ["pretrain", "from-yaml", "pretrain.yaml"])
    assert r.exit_code == 0, r.output + str(r.exception)
    run = next((tmp_path / "ckpt").glob("run-*"))
    ck = sorted(p.name for p in run.glob("checkpoint-*"))
    assert ck == ["checkpoint-12", "checkpoint-3", "checkpoint-6", "checkpoint-9"]
    for f in ("pytorch_model.bin", "optimizer.pt", "scheduler.pt", "rng_state.pth", "training_state.json"):
        assert (run / "checkpoint-6" / f).exists()
    assert json.loads((run / "checkpoint-6" / "training_state.json").read_text())["global_step"] == 6
    lines = [json.loads(l) for l in (run / "metrics.jsonl").read_text().splitlines()]
    assert any("eval/loss" in l for l in lines) and any("train/tokens_per_sec" in l for l in lines)

    # resume from step 6 with one extra epoch: continues in the same run dir, later checkpoints archived
    cfg["resume"] = {"is_resume": True, "checkpoint_dir": str(run / "checkpoint-6"), "extra_epochs": 1}
    (tmp_path / "pretrain.yaml").write_text(yaml.safe_dump(cfg))
    r = runner.invoke(cli, ["pretrain", "from-yaml", "pretrain.yaml"])
    assert r.exit_code == 0, r.output + str(r.exception)
    assert (run / ".resume_counter").read_text() == "1"
    archived = list(run.glob("archived_*"))
    assert len(archived) == 1 and sorted(p.name for p in archived[0].iterdir()) == ["checkpoint-12", "checkpoint-9"]
    assert (run / "checkpoint-18").exists()                                            # 3 epochs x 6 steps

    # pure_torch.enabled: false = the reference's HF-Trainer recipe: padded batches, HF files in the checkpoints
    hf = {k: (dict(v) if isinstance(v, dict) else v) for k, v in cfg.items()}
    hf["resume"] = {"is_resume": False, "checkpoint_dir": "", "extra_epochs": None}
    hf["pure_torch"] = {"enabled": False}
    hf["pretraining"].update(ckp_dir="ckpt_hf", num_epochs=1, save_steps=3)
    (tmp_path / "hf.yaml").write_text(yaml.safe_dump(hf))
    r = runner.invoke(cli, ["pretrain", "from-yaml", "hf.yaml"])
    assert r.exit_code == 0, r.output + str(r.exception)
    hf_run = next((tmp_path / "ckpt_hf").glob("run-*"))
    some = sorted(hf_run.glob("checkpoint-*"))[0]
    for f in ("model.safetensors", "trainer_state.json", "pytorch_model.bin", "optimizer.pt"):
        assert (some / f).exists(), f

    bad = dict(cfg)
    bad["pretraining"] = {**cfg["pretraining"], "gradient_accumulation_steps": 2}
    (tmp_path / "bad.yaml").write_text(yaml.safe_dump(bad))
    r = runner.invoke(cli, ["pretrain", "from-yaml", "bad.yaml"])
    assert r.exit_code != 0 and "inferred" in r.output
    assert runner.invoke(cli, ["pretrain", "from-yaml", "missing.yaml"]).exit_code != 0


def test_cli_distillation_on_the_fly(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    runner = CliRunner()
    _write_params(tmp_path, "distillation", on_the_fly=True)
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "builtin"])
    assert r.exit_code == 0, r.output
    assert yaml.safe_load((tmp_path / "out" / "kd" / ".data_manifest").read_text())["on_the_fly"] is True
    assert runner.invoke(cli, ["distill", "get-yaml", "distill.yaml"]).exit_code == 0
    cfg = yaml.safe_load((tmp_path / "distill.yaml").read_text())
    cfg["model"].update(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2)
    cfg["distillation"].update(dataset_dir="out/kd", ckp_dir="dckpt", num_epochs=2, batch_size=8, logging_steps=1,
                               eval_steps=4, save_steps=6, bf16=False, teacher_random_init=True,
                               teacher={"d_model": 1024, "d_kv": 16, "d_ff": 64, "num_layers": 1, "num_heads": 4})
    (tmp_path / "distill.yaml").write_text(yaml.safe_dump(cfg))
    r = runner.invoke(cli, ["distill", "from-yaml", "distill.yaml"])
    assert r.exit_code == 0, r.output + str(r.exception)
    run = next((tmp_path / "dckpt").glob("run-*"))
    assert (run / "training_config.json").exists() and (run / "model.safetensors").exists()
    assert (run / "checkpoint-6" / "model.safetensors").exists() and (run / "checkpoint-12" / "optimizer.pt").exists()
    lines = [json.loads(l) for l in (run / "metrics.jsonl").read_text().splitlines()]
    train = [l["train/loss"] for l in lines if "train/loss" in l]
    assert train[-1] < train[0]

    # `distill run --resume-from` without --dataset-dir: the dataset comes back from the run's
    # training_config.json, here reduced to the flat keys the reference writes
    # (distillation/pipeline.py:557-576, cli/distill.py:406-425)
    from nanoplm_b200.config import schema
    from nanoplm_b200.runtime.distill import REFERENCE_TRAINING_CONFIG_KEYS
    saved = json.loads((run / "training_config.json").read_text())
    assert all(k in saved for k in REFERENCE_TRAINING_CONFIG_KEYS) and saved["on_the_fly"] is True
    flat = {k: saved[k] for k in REFERENCE_TRAINING_CONFIG_KEYS}
    flat["train_h5_prefix"] = flat["val_h5_prefix"] = "None"
    (run / "training_config.json").write_text(json.dumps(flat))
    monkeypatch.setattr(schema.TeacherConfig.__init__, "__defaults__",
                        (128, 1024, 16, 64, 1, 4, 32, 128, 1e-6, "tiny-random"))
    args = ["distill", "run", "--resume-from", str(run / "checkpoint-6"), "--extra-epochs", "1", "--ckp-dir", "dckpt",
            "--num-epochs", "2", "--batch-size", "8", "--logging-steps", "1", "--eval-steps", "4", "--save-steps", "6",
            "--no-bf16", "--teacher-random-init", "--hidden-size", "64", "--intermediate-size", "128",
            "--num-hidden-layers", "2", "--num-attention-heads", "2", "--no-threading"]
    r = runner.invoke(cli, args)
    assert r.exit_code == 0, r.output + str(r.exception)
    assert (run / "checkpoint-18").exists() and (run / ".resume_counter").read_text() == "1"
    (run / "training_config.json").unlink()
    r = runner.invoke(cli, args)
    assert r.exit_code != 0 and "training_config.json not found" in r.output


def test_cli_data_single_steps_with_the_reference_option_spellings(tmp_path, monkeypatch):
    """The single-step `data` commands with the option names, defaults and output conventions of the
    reference CLI (cli/data.py:34-625): a directory as download target, "already exists" reported
    with exit code 0, `--output` for split / save-pretrain-dataset, a directory and `--skip-n` for
    save-kd-dataset, `--input-file / --n-shards / --total-sequences` for shard."""
    import gzip
    monkeypatch.chdir(tmp_path)
    runner = CliRunner()
    src = write_synthetic_fasta(tmp_path / "src" / "mini.fasta", 40, 12, 60, seed=2)
    with open(src, "rb") as f, gzip.open(tmp_path / "src" / "mini.fasta.gz", "wb") as g:
        g.write(f.read())
    url = (tmp_path / "src" / "mini.fasta.gz").as_uri()

    r = runner.invoke(cli, ["data", "download", "--url", url])                     # default: ./downloaded_dataset/
    assert r.exit_code == 0, r.output
    got = tmp_path / "downloaded_dataset" / "mini.fasta.gz"
    assert got.read_bytes() == (tmp_path / "src" / "mini.fasta.gz").read_bytes()
    r = runner.invoke(cli, ["data", "download", "--url", url])
    assert r.exit_code == 0 and "already exists" in r.output
    assert runner.invoke(cli, ["data", "download", "--url", url, "-f", "-o", "downloaded_dataset"]).exit_code == 0
    assert runner.invoke(cli, ["data", "download", "swissprot", "--url", url]).exit_code == 2
    assert runner.invoke(cli, ["data", "download"]).exit_code == 2
    assert runner.invoke(cli, ["data", "download", "-h"]).exit_code == 0

    assert runner.invoke(cli, ["data", "extract", "-i", str(got), "-o", "raw/mini.fasta"]).exit_code == 0
    assert runner.invoke(cli, ["data", "shuffle", "-i", "raw/mini.fasta", "-o", "raw/shuf.fasta"]).exit_code == 0
    r = runner.invoke(cli, ["data", "filter", "-i", "raw/shuf.fasta", "-o", "raw/filt.fasta", "--min-seq-len", "15"])
    assert r.exit_code == 0, r.output
    r = runner.invoke(cli, ["data", "split", "-i", "raw/filt.fasta", "--output", "split", "--val-ratio", "0.25"])
    assert r.exit_code == 0 and (tmp_path / "split" / "train.fasta").exists() and (tmp_path / "split" / "val.fasta").exists()
    r = runner.invoke(cli, ["data", "save-pretrain-dataset", "-i", "split/train.fasta", "--output", "shards/train",
                            "--samples-per-shard", "10", "--max-seq-len", "64"])
    assert r.exit_code == 0, r.output
    assert len(list((tmp_path / "shards" / "train").glob("*.bin"))) >= 2
    assert runner.invoke(cli, ["data", "save-pretrain-dataset", "-i", "split/train.fasta", "--output", "shards/train",
                               "--max-seq-len", "64"]).exit_code != 0          # exists: needs -f
    assert runner.invoke(cli, ["data", "save-pretrain-dataset", "-i", "split/train.fasta", "--output", "shards/train",
                               "--max-seq-len", "64", "-f"]).exit_code == 0

    from nanoplm_b200.data.fasta import count_fasta
    from nanoplm_b200.data.kd_dataset import count_kd_sequences
    n_val = count_fasta(tmp_path / "split" / "val.fasta")
    # the tiny random teacher of the tests instead of the 1.2 B parameter default
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.models import teacher as teacher_mod
    small = TeacherConfig(d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4)
    monkeypatch.setattr(teacher_mod.T5EncoderTeacher.__init__, "__defaults__", (small, True, 0))
    r = runner.invoke(cli, ["data", "save-kd-dataset", "-i", "split/val.fasta", "-o", "kd", "--max-seq-len", "64",
                            "--skip-n", "2", "--teacher-random-init", "--device", "cpu"])
    assert r.exit_code == 0, r.output + str(r.exception)
    files = sorted((tmp_path / "kd").glob("val_kd_dataset.*"))
    assert len(files) == 1 and count_kd_sequences(files[0]) == n_val - 2
    assert runner.invoke(cli, ["data", "save-kd-dataset", "-i", "split/val.fasta", "-o", "kd/x.txt"]).exit_code != 0
    assert runner.invoke(cli, ["data", "save-kd-dataset", "-i", "split/val.fasta", "-o", "kd", "--samples-per-shard",
                               "0"]).exit_code != 0
    r = runner.invoke(cli, ["data", "shard", "--input-file", str(files[0]), "--n-shards", "2", "-o", "kd_parts",
                            "--total-sequences", str(n_val - 2)])
    assert r.exit_code == 0, r.output + str(r.exception)
    assert sum(count_kd_sequences(p) for p in (tmp_path / "kd_parts").iterdir()) == n_val - 2


def test_cli_pretrain_run_with_options(tmp_path, monkeypatch):
    """`pretrain run` takes the settings as options (the reference's spellings included:
    --adam-warmup-ratio, --compile / --no-compile, --use-packing / --no-packing) and, with
    --no-pure-torch, runs the HF-Trainer recipe."""
    from nanoplm_b200.data.synthetic import write_synthetic_dataset
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    write_synthetic_dataset(tmp_path / "ds", 64, 16, 10, 60, samples_per_shard=32)
    runner = CliRunner()
    base = ["pretrain", "run", "--dataset-dir", "ds", "--micro-batch-size", "8", "--global-batch-size", str(8 * 64),
            "--num-epochs", "1", "--logging-steps", "1", "--eval-steps", "4", "--save-steps", "2", "--num-workers", "0",
            "--no-bf16", "--hidden-size", "32", "--intermediate-size", "64", "--num-hidden-layers", "1",
            "--num-attention-heads", "2", "--max-position-embeddings", "64", "--adam-warmup-ratio", "0.25",
            "--no-compile"]
    r = runner.invoke(cli, base + ["--ckp-dir", "a", "--use-packing", "--target-packed-rows", "3"])
    assert r.exit_code == 0, r.output + str(r.exception)
    run = next((tmp_path / "a").glob("run-*"))
    # 64 sequences / 8 per micro-batch / 2 micro-batches per step = 4 steps, one of them warm-up
    assert (run / "checkpoint-4" / "pytorch_model.bin").exists() and not (run / "checkpoint-4" / "model.safetensors").exists()
    lines = [json.loads(l) for l in (run / "metrics.jsonl").read_text().splitlines() if "train/learning_rate" in l]
    assert [l["train/learning_rate"] for l in lines[:2]] == [0.0, pytest.approx(1e-3)]
    r = runner.invoke(cli, base + ["--ckp-dir", "b", "--no-packing", "--no-pure-torch"])
    assert r.exit_code == 0, r.output + str(r.exception)
    run = next((tmp_path / "b").glob("run-*"))
    assert (run / "checkpoint-4" / "model.safetensors").exists() and (run / "checkpoint-4" / "trainer_state.json").exists()
    r = runner.invoke(cli, base + ["--ckp-dir", "b", "--resume-from", str(run / "checkpoint-2"), "--extra-epochs", "1"])
    assert r.exit_code == 0, r.output + str(r.exception)
    assert (run / "checkpoint-8").exists() and len(list(run.glob("archived_*"))) == 1
    assert runner.invoke(cli, base + ["--optimizer", "sgd"]).exit_code == 2


def test_loader_error_branches_and_coercions(tmp_path):
    """What the strict loaders refuse and what they coerce (reference: cli/pretrain.py:742-924,
    cli/distill.py:629-743): strings for numbers and booleans are converted, anything else is named
    in the error."""
    from nanoplm_b200.config.loaders import (load_distill_config, load_student_config, read_yaml)
    base = yaml.safe_load(PRETRAIN_YAML)
    pre = dict(base["pretraining"])
    cfg = load_pretrain_config({**pre, "bf16": "yes", "tf32": 0, "micro_batch_size": "16", "global_batch_size": "2e6",
                                "adam_learning_rate": "5e-4", "muon_nesterov": "FALSE"})
    assert cfg.bf16 is True and cfg.tf32 is False and cfg.micro_batch_size == 16 and cfg.global_batch_size == 2_000_000
    assert cfg.adam_learning_rate == 5e-4 and cfg.muon_nesterov is False
    for key, bad, msg in (("bf16", "maybe", "Invalid boolean"), ("micro_batch_size", "many", "Must be an integer"),
                          ("micro_batch_size", 2.5, "Must be an integer"), ("logging_steps", [1], "Must be an integer")):
        with pytest.raises(ConfigError, match=msg):
            load_pretrain_config({**pre, key: bad})
    with pytest.raises(ConfigError, match="required"):
        load_pretrain_config(None)
    with pytest.raises(ConfigError, match="required"):
        load_model_config(None)
    with pytest.raises(ConfigError, match="model.moe"):
        load_model_config({**base["model"], "moe": {"num_experts": 8, "nope": 1}})
    both = load_pretrain_config({**pre, "learning_rate": 1e-3, "adam_learning_rate": "1e-3"})      # same value twice: fine
    assert both.adam_learning_rate == 1e-3
    assert load_pretrain_config({**pre, "learning_rate": 2e-3, "adam_learning_rate": 1e-3}).adam_learning_rate == 1e-3
    with pytest.raises(ConfigError, match="Unexpected resume"):
        load_resume_config({"is_resume": False, "nope": 1})

    dis = yaml.safe_load(DISTILL_YAML)
    with pytest.raises(ConfigError, match="required"):
        load_student_config(None)
    with pytest.raises(ConfigError, match="Unexpected model"):
        load_student_config({**dis["model"], "nope": 1})
    with pytest.raises(ConfigError, match="required"):
        load_distill_config(None)
    d = {**dis["distillation"], "dataset_dir": "x"}
    with pytest.raises(ConfigError, match="dataset_dir is required"):
        load_distill_config({k: v for k, v in d.items() if k != "dataset_dir"})
    assert load_distill_config({k: v for k, v in d.items() if k != "dataset_dir"}, require_dataset_dir=False).dataset_dir is None
    with pytest.raises(ConfigError, match="Unexpected distillation configuration"):
        load_distill_config({**d, "nope": 1})
    with pytest.raises(ConfigError, match="distillation.teacher"):
        load_distill_config({**d, "teacher": {"d_model": 64, "nope": 1}})
    got = load_distill_config({**d, "lr_scheduler_kwargs": '{"num_warmup_steps": 5}', "teacher": {"d_model": "64"},
                               "learning_rate": "3e-4", "use_threading": "false"})
    assert got.lr_scheduler_kwargs == {"num_warmup_steps": 5} and got.teacher.d_model == 64
    assert got.learning_rate == 3e-4 and got.use_threading is False

    with pytest.raises(FileNotFoundError):
        read_yaml(tmp_path / "missing.yaml")
    (tmp_path / "list.yaml").write_text("- 1\n- 2\n")
    with pytest.raises(ConfigError, match="mapping"):
        read_yaml(tmp_path / "list.yaml")


def test_cli_data_from_yaml_with_the_dvc_runner(tmp_path, monkeypatch):
    """The dvc runner of `data from-yaml` (reference: cli/data.py:926-979), against a stand-in `dvc`
    executable that records its arguments: `dvc init` happens once (--no-scm outside a git work
    tree) unless --no-auto-init, `dvc repro` gets -f / -v / the target, a failing repro is reported, and
    the in-process part (shards + manifest) follows."""
    import stat
    monkeypatch.chdir(tmp_path)
    runner = CliRunner()
    _write_params(tmp_path, "pretrain")
    (tmp_path / "dvc.yaml").write_text("stages: {}\n")
    # what the dvc stages would have produced
    from nanoplm_b200.data.fasta import iter_fasta, write_fasta
    recs = list(iter_fasta(tmp_path / "raw" / "x.fasta"))
    write_fasta(recs[:40], tmp_path / "raw" / "split" / "train.fasta")
    write_fasta(recs[40:50], tmp_path / "raw" / "split" / "val.fasta")
    bindir = tmp_path / "bin"
    bindir.mkdir()
    log = tmp_path / "dvc_calls.txt"
    fake = bindir / "dvc"
    fake.write_text(f"#!/bin/sh\necho \"$@\" >> {log}\nif [ \"$1\" = init ]; then mkdir -p .dvc; fi\n"
                    f"if [ -f {tmp_path}/fail_repro ] && [ \"$1\" = repro ]; then exit 3; fi\nexit 0\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(bindir) + os.pathsep + os.environ["PATH"])
    monkeypatch.setenv("GIT_CEILING_DIRECTORIES", str(tmp_path.parent))      # tmp_path is not inside a git work tree

    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "dvc", "--no-auto-init"])
    assert r.exit_code != 0 and "DVC is not initialized" in r.output
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "dvc", "--force", "--verbose"])
    assert r.exit_code == 0, r.output + str(r.exception)
    calls = log.read_text().splitlines()
    assert calls == ["init -q --no-scm", "repro -v -f split"]
    manifest = yaml.safe_load((tmp_path / "out" / "shards" / ".data_manifest").read_text())
    assert manifest["train_sequences"] == 40 and manifest["val_sequences"] == 10
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--target", "filter"])     # auto: dvc + dvc.yaml present
    assert r.exit_code == 0 or "already exist" in r.output
    assert log.read_text().splitlines()[-1] == "repro filter" and len(log.read_text().splitlines()) == 3   # no second init
    (tmp_path / "fail_repro").write_text("")
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "dvc"])
    assert r.exit_code != 0 and "dvc repro failed with exit code 3" in r.output
    monkeypatch.setenv("PATH", str(tmp_path / "nothing"))
    r = runner.invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "dvc"])
    assert r.exit_code != 0 and "'dvc' command not found" in r.output
