"""`run_distillation` end to end on two CPU ranks (gloo), in both dataset modes, with sequence counts
that do not divide by world x batch, so ranks that disagreed on the number of collectives (or a
rank-0-only gather at the end of the run) would show up as a hang / time-out here. Also: a
checkpoint taken in the middle of an epoch resumes at the same place."""
import json
import os
import socket
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import yaml
from click.testing import CliRunner

from nanoplm_b200.cli import cli
from nanoplm_b200.config.templates import PARAMS_YAML
from nanoplm_b200.data.synthetic import write_synthetic_fasta

TEACHER = {"d_model": 1024, "d_kv": 16, "d_ff": 64, "num_layers": 1, "num_heads": 4}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _prepare(tmp: Path, on_the_fly: bool) -> None:
    params = yaml.safe_load(PARAMS_YAML)
    # 67 sequences -> 54 train / 13 val: neither divides by 2 ranks x batch 8
    params["data_params"].update(pipeline_mode="distillation", seqs_num=67, min_seq_len=10, max_seq_len=48,
                                 val_ratio=0.2)
    params["distillation_config"].update(output_dir="out/kd", on_the_fly=on_the_fly, samples_per_shard=16,
                                         teacher_random_init=True, embed_calc_batch_size=8)
    params["data_dirs"].update(url="unused", compressed_fasta="raw/x.fasta.gz", extracted_fasta="raw/x.fasta",
                               shuffled_fasta="raw/x_shuf.fasta", filtered_fasta="raw/x_filt.fasta",
                               splitted_fasta_dir="raw/split")
    (tmp / "params.yaml").write_text(yaml.safe_dump(params))
    write_synthetic_fasta(tmp / "raw" / "x.fasta", 120, 5, 60, seed=11)
    cwd = os.getcwd()
    os.chdir(tmp)
    try:
        r = CliRunner().invoke(cli, ["data", "from-yaml", "params.yaml", "--runner", "builtin"])
    finally:
        os.chdir(cwd)
    assert r.exit_code == 0, r.output


def _rank_main(rank, world, port, tmp, resume_from, max_steps, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), WANDB_MODE="disabled")
    os.chdir(tmp)
    torch.set_num_threads(1)
    from nanoplm_b200.config.schema import DistillationConfig, ResumeConfig, StudentConfig
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    from nanoplm_b200.runtime.distill import run_distillation
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = DistillationConfig(dataset_dir="out/kd", ckp_dir="dckpt", num_epochs=2, batch_size=8, logging_steps=1,
                             eval_steps=3, save_steps=3, bf16=False, multi_gpu=True, world_size=world,
                             gradient_accumulation_steps=2, teacher_random_init=True, teacher=dict(TEACHER))
    model = StudentConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2)
    resume = ResumeConfig(is_resume=True, checkpoint_dir=resume_from) if resume_from else None
    out = run_distillation(model, cfg, resume, max_steps=max_steps)
    if rank == 0:
        q.put({"global_step": out["global_step"], "losses": out["losses"], "output_dir": out["output_dir"]})
    dist.destroy_process_group()


def _run(tmp, world, resume_from=None, max_steps=None):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, str(tmp), resume_from, max_steps, q))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    assert not hung, "a rank never finished: the ranks disagree on their collectives"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return q.get()


@pytest.mark.parametrize("on_the_fly", [True, False], ids=["on_the_fly", "precomputed"])
def test_two_rank_distillation_runs_to_completion_and_resumes(tmp_path, on_the_fly):
    _prepare(tmp_path, on_the_fly)
    res = _run(tmp_path, 2)
    run = Path(tmp_path) / res["output_dir"] if not os.path.isabs(res["output_dir"]) else Path(res["output_dir"])
    assert res["global_step"] >= 4
    assert (run / "model.safetensors").exists() or (run / "pytorch_model.bin").exists()
    assert (run / "checkpoint-3" / "optimizer.pt").exists()
    first = [l for _, l in res["losses"]]
    assert first[-1] < first[0]
    # resume from the mid-epoch checkpoint (step 3 of an epoch of 2 optimizer steps): one more step
    # continues at global step 4 instead of replaying the epoch
    res2 = _run(tmp_path, 2, resume_from=str(run / "checkpoint-3"), max_steps=4)
    assert res2["global_step"] == 4
    assert json.loads((Path(res2["output_dir"]) / "checkpoint-4" / "trainer_state.json").read_text()
                      if os.path.isabs(res2["output_dir"]) else
                      (Path(tmp_path) / res2["output_dir"] / "checkpoint-4" / "trainer_state.json").read_text()
                      )["global_step"] == 4


def test_stored_embeddings_from_explicit_paths_with_heartbeat_and_mid_epoch_resume(tmp_path, monkeypatch):
    """One process, no dataset directory: the explicit embedding-file prefixes of the configuration
    (how a run resumed through the reference's `training_config.json` arrives, cli/distill.py:406-425),
    heartbeat files while training, and a resume from a checkpoint in the middle of an epoch."""
    from nanoplm_b200.config.schema import DistillationConfig, ResumeConfig, StudentConfig, TeacherConfig
    from nanoplm_b200.data.kd_dataset import SaveKDDataset
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    from nanoplm_b200.runtime.distill import run_distillation
    from nanoplm_b200.runtime.watchdog import read_heartbeat
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    teacher = T5EncoderTeacher(TeacherConfig(d_model=1024, d_kv=8, d_ff=32, num_layers=1, num_heads=2))
    for split, n in (("train", 40), ("val", 8)):
        fasta = write_synthetic_fasta(tmp_path / f"{split}.fasta", n, 8, 20, seed=5)
        SaveKDDataset(fasta, tmp_path / "kd" / split / f"{split}_kd.kdz", max_seq_len=24, batch_size=8, device="cpu",
                      samples_per_shard=16, teacher=teacher).run()
    model = StudentConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2)

    def cfg():
        return DistillationConfig(dataset_dir=None, train_h5_prefix=str(tmp_path / "kd" / "train" / "train_kd.kdz"),
                                  val_h5_prefix=str(tmp_path / "kd" / "val" / "val_kd.kdz"), max_seq_len=24,
                                  on_the_fly=False, ckp_dir="ck", num_epochs=2, batch_size=8, logging_steps=1,
                                  eval_steps=100, save_steps=3, bf16=False, heartbeat_seconds=0.2)
    res = run_distillation(model, cfg())
    run = Path(res["output_dir"])
    assert res["global_step"] == 10 and (run / "checkpoint-3").exists() and (run / "checkpoint-9").exists()   # 5 steps per epoch
    beat = read_heartbeat(run / "heartbeat" / "rank-0")
    assert beat is not None and beat[1] == 10
    first = dict(res["losses"])
    with pytest.raises(ValueError, match="dataset_dir is required unless"):
        run_distillation(model, DistillationConfig(dataset_dir=None, on_the_fly=False, ckp_dir="ck2"))
    # checkpoint-3 lies inside the first epoch: the resumed run skips three micro-batches and sees the same data
    res2 = run_distillation(model, cfg(), ResumeConfig(True, str(run / "checkpoint-3"), None))
    again = dict(res2["losses"])
    assert res2["global_step"] == 10 and sorted(again) == list(range(4, 11))
    assert all(abs(again[s] - first[s]) < 1e-4 * max(1.0, abs(first[s])) for s in again), (first, again)
