"""Elastic recovery on CPU ranks (gloo): the supervisor restarts a job from its latest complete
checkpoint after a rank dies, raises or stops making progress. Failures are injected on the host,
between optimizer steps (`NPLM_INJECT_FAULT`); nothing here touches a GPU."""
import json
import os
import sys
from pathlib import Path

import pytest
import yaml

from nanoplm_b200.config.templates import PRETRAIN_YAML
from nanoplm_b200.data.synthetic import write_synthetic_dataset
from nanoplm_b200.runtime.supervisor import Supervisor

ROOT = Path(__file__).resolve().parent.parent


def _config(tmp: Path, **pre) -> Path:
    write_synthetic_dataset(tmp / "ds", 96, 16, 10, 60, samples_per_shard=48)
    cfg = yaml.safe_load(PRETRAIN_YAML)
    cfg["model"].update(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                        max_position_embeddings=64)
    cfg["pretraining"].update(dataset_dir=str(tmp / "ds"), ckp_dir=str(tmp / "ckpt"), micro_batch_size=8,
                              global_batch_size=8 * 64 * 2, num_epochs=2, logging_steps=1, eval_steps=100,
                              save_steps=2, num_workers=0, bf16=False, fused_comm=False)
    cfg["pretraining"].update(pre)
    cfg["pure_torch"].update(use_packing=False)
    path = tmp / "pretrain.yaml"
    path.write_text(yaml.safe_dump(cfg))
    return path


def _env():
    return {"WANDB_MODE": "disabled", "PYTHONPATH": str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""),
            "CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "2"}


def _steps(run: Path) -> list[int]:
    lines = [json.loads(l) for l in (run / "metrics.jsonl").read_text().splitlines()]
    return [l["train/global_step"] for l in lines if "train/loss" in l]


@pytest.mark.timeout(600)
def test_job_restarts_from_the_latest_checkpoint_after_a_rank_dies(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    cfg = _config(tmp_path)
    # rank 1 of 2 is killed (exit code 17) right after step 3 of the first attempt; checkpoint-2 exists then
    sup = Supervisor(cfg, nproc=2, max_restarts=2, grace_seconds=5, log_dir=tmp_path / "logs",
                     extra_env={**_env(), "NPLM_INJECT_FAULT": "1:3:exit:0"})
    assert sup.run() == 0, [a.__dict__ for a in sup.attempts]
    assert sup.restarts == 1
    first, second = sup.attempts
    assert first.exit_codes[1] == 17 and "1 exited with code 17" in first.reason
    # the survivor was ended by the supervisor, or noticed the lost connection itself just before
    assert first.exit_codes[0] not in (0, None)
    assert second.resumed_from.endswith("checkpoint-2") and second.exit_codes == [0, 0]
    run = Path(second.run_dir)
    assert run == Path(first.run_dir) and len(list((tmp_path / "ckpt").glob("run-*"))) == 1
    steps = _steps(run)
    total = steps[-1]
    # rank 0 was waiting for rank 1 in the statistics exchange of step 3 when the attempt ended: steps 1-2
    # come from the first attempt, 3 onwards (redone from checkpoint-2) from the second
    assert total == 6 and steps == list(range(1, total + 1))
    assert "[step 3/" not in (tmp_path / "logs" / "attempt-0-rank-0.log").read_text()
    assert (run / f"checkpoint-{total}").exists() and (run / ".resume_counter").read_text().strip() == "1"
    log = (tmp_path / "logs" / "attempt-1-rank-0.log").read_text()
    assert "Resumed at global_step=2" in log


@pytest.mark.timeout(600)
def test_exception_before_any_checkpoint_starts_over_and_repeated_failures_give_up(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    cfg = _config(tmp_path, save_steps=100)
    # a single rank raises after step 1: nothing has been saved, so the second attempt is a fresh run
    sup = Supervisor(cfg, nproc=1, max_restarts=1, log_dir=tmp_path / "logs",
                     extra_env={**_env(), "NPLM_INJECT_FAULT": "0:1:raise:0"})
    assert sup.run() == 0
    assert sup.restarts == 1 and sup.attempts[1].resumed_from is None
    assert sup.attempts[0].exit_codes == [1] and "InjectedFault" in (tmp_path / "logs" / "attempt-0-rank-0.log").read_text()
    # a failure on every attempt: the supervisor stops after max_restarts and reports it
    always = Supervisor(cfg, nproc=1, max_restarts=1, command=[sys.executable, "-c", "import sys; sys.exit(3)"],
                        extra_env=_env())
    assert always.run() == 1 and len(always.attempts) == 2 and always.attempts[-1].exit_codes == [3]


@pytest.mark.timeout(600)
def test_a_rank_that_stops_making_progress_is_ended_and_the_job_resumes(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    cfg = _config(tmp_path, heartbeat_seconds=0.5)
    # the only rank stays alive but stops stepping after step 3 (its heartbeat keeps beating)
    sup = Supervisor(cfg, nproc=1, max_restarts=1, stall_seconds=12, grace_seconds=3, log_dir=tmp_path / "logs",
                     extra_env={**_env(), "NPLM_INJECT_FAULT": "0:3:stall:0"})
    assert sup.run() == 0, [a.__dict__ for a in sup.attempts]
    assert sup.restarts == 1 and "no progress on ranks [0]" in sup.attempts[0].reason
    assert sup.attempts[0].exit_codes[0] not in (0, None)
    assert sup.attempts[1].resumed_from.endswith("checkpoint-2")
    run = Path(sup.attempts[1].run_dir)
    assert _steps(run)[-1] == max(_steps(run)) and (run / f"checkpoint-{_steps(run)[-1]}").exists()


def test_supervise_command_is_wired(tmp_path, monkeypatch):
    from click.testing import CliRunner

    from nanoplm_b200.cli import cli
    monkeypatch.chdir(tmp_path)
    r = CliRunner().invoke(cli, ["pretrain", "supervise", "missing.yaml"])
    assert r.exit_code != 0 and "Config file not found" in r.output
    r = CliRunner().invoke(cli, ["pretrain", "supervise", "--help"])
    assert r.exit_code == 0 and "--max-restarts" in r.output and "--nproc" in r.output


@pytest.mark.timeout(600)
def test_distillation_job_restarts_after_a_rank_raises(tmp_path, monkeypatch):
    from nanoplm_b200.config.templates import DISTILL_YAML
    from nanoplm_b200.data.manifest import DistillationManifest, write_manifest
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    monkeypatch.chdir(tmp_path)
    kd = tmp_path / "kd"
    write_synthetic_fasta(kd / "train.fasta", 64, 10, 40, seed=1)
    write_synthetic_fasta(kd / "val.fasta", 16, 10, 40, seed=2)
    write_manifest(kd, DistillationManifest(
        pipeline_mode="distillation", seqs_num=80, min_seq_len=10, max_seq_len=48, val_ratio=0.2, train_dir=".",
        val_dir=".", train_sequences=64, val_sequences=16, teacher_model="prott5", on_the_fly=True,
        train_fasta="train.fasta", val_fasta="val.fasta"))
    cfg = yaml.safe_load(DISTILL_YAML)
    cfg["model"].update(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2)
    cfg["distillation"].update(dataset_dir=str(kd), ckp_dir=str(tmp_path / "dckpt"), num_epochs=2, batch_size=8,
                               logging_steps=1, eval_steps=100, save_steps=2, bf16=False, fused_comm=False,
                               teacher_random_init=True,
                               teacher={"d_model": 1024, "d_kv": 8, "d_ff": 32, "num_layers": 1, "num_heads": 2})
    path = tmp_path / "distill.yaml"
    path.write_text(yaml.safe_dump(cfg))
    sup = Supervisor(path, nproc=2, max_restarts=2, grace_seconds=5, log_dir=tmp_path / "logs", section="distillation",
                     extra_env={**_env(), "NPLM_INJECT_FAULT": "1:3:raise:0"})
    assert sup.run() == 0, [a.__dict__ for a in sup.attempts]
    assert sup.restarts == 1 and sup.attempts[1].resumed_from.endswith("checkpoint-2")
    assert sup.attempts[0].exit_codes[1] == 1 and sup.attempts[1].exit_codes == [0, 0]
    run = Path(sup.attempts[1].run_dir)
    steps = _steps(run)
    # 2 epochs x 4 steps; what the first attempt logged past checkpoint-2 shows up again from the second
    assert steps[-1] == 8 and sorted(set(steps)) == list(range(1, 9)) and (run / "checkpoint-8").exists()
    assert steps[steps.index(2) + 1:].count(3) >= 1 and steps == sorted(steps)
    assert (run / "model.safetensors").exists()


@pytest.mark.timeout(300)
def test_sigterm_to_the_supervisor_ends_the_ranks(tmp_path):
    """The ranks run in sessions of their own; a SIGTERM to the supervising process still ends them."""
    import signal
    import subprocess
    import time
    cfg = tmp_path / "c.yaml"
    cfg.write_text("pretraining: {ckp_dir: ck}\n")
    pidfile = tmp_path / "rank.pid"
    child = f"import os, time; open({str(pidfile)!r}, 'w').write(str(os.getpid())); time.sleep(120)"
    code = ("import sys; from nanoplm_b200.runtime.supervisor import Supervisor; "
            f"sys.exit(Supervisor({str(cfg)!r}, nproc=1, max_restarts=0, grace_seconds=2, "
            f"command=[sys.executable, '-c', {child!r}]).run())")
    sup = subprocess.Popen([sys.executable, "-c", code], cwd=tmp_path, env={**os.environ, **_env()})
    deadline = time.time() + 120
    while not pidfile.exists() or not pidfile.read_text():
        assert time.time() < deadline and sup.poll() is None
        time.sleep(0.2)
    rank_pid = int(pidfile.read_text())
    sup.send_signal(signal.SIGTERM)
    assert sup.wait(timeout=60) == 128 + signal.SIGTERM
    for _ in range(100):
        try:
            os.kill(rank_pid, 0)
        except ProcessLookupError:
            break
        time.sleep(0.1)
    else:
        os.kill(rank_pid, signal.SIGKILL)          # this exact process, started above
        raise AssertionError("the rank outlived its supervisor")
