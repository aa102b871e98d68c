"""Embedding distillation (`nanoplm distill from-yaml`): the ProtX student regresses the per-residue
embeddings of a frozen T5-style teacher with a masked MSE
(reference: src/nanoplm/distillation/pipeline.py:457-754, trainer.py:7-49, collator.py:6-111).

Differences from the reference by design: the teacher runs on the training GPU inside the step and
its output stays on the device (the reference computes it in the collator and ships it GPU -> CPU
fp32 -> GPU every step); data parallelism uses the sharded engine of the pretraining pipeline (the
teacher is excluded from it and replicated); checkpoints are `checkpoint-N/{model.safetensors,
optimizer.pt, scheduler.pt, trainer_state.json}` plus `<run>/training_config.json`.
"""
from __future__ import annotations

import json
import math
import os
import time
from pathlib import Path
from typing import Optional

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from nanoplm_b200.config.schema import DistillationConfig, ResumeConfig, StudentConfig, as_plain_dict
from nanoplm_b200.data.kd_dataset import KDDatasetOnTheFly, LoadKDDataset
from nanoplm_b200.data.manifest import DistillationManifest, get_dataset_paths
from nanoplm_b200.data.tokenizer import StudentTokenizer, TeacherTokenizer
from nanoplm_b200.data.validation import validate_distillation_dataset
from nanoplm_b200.models.student import ProtX
from nanoplm_b200.ops import functional as ops
from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
from nanoplm_b200.runtime.metrics import MetricsSink
from nanoplm_b200.runtime.pretrain import ResumableDistributedSampler, init_distributed, set_seed
from nanoplm_b200.runtime.run_dirs import prepare_run_and_steps
from nanoplm_b200.runtime.schedule import make_distill_schedule
from nanoplm_b200.utils.logging import logger


class DistillDataCollator:
    """Pre-computed mode: stacks stored tensors. On-the-fly mode: tokenises raw sequences for the
    student and for the teacher, both padded to max_seq_len (the teacher forward happens in the
    training step, on the device)."""

    def __init__(self, on_the_fly: bool, max_seq_len: int):
        self.on_the_fly, self.max_seq_len = on_the_fly, max_seq_len
        self.student_tok, self.teacher_tok = StudentTokenizer(), TeacherTokenizer()

    def __call__(self, examples: list[dict]) -> dict:
        if not self.on_the_fly:
            return {k: torch.stack([e[k] for e in examples]) for k in
                    ("input_ids", "attention_mask", "teacher_embeddings")}
        seqs = [e["raw_sequence"] for e in examples]
        L = self.max_seq_len
        st = self.student_tok(seqs, padding="max_length", max_length=L, truncation=True, return_tensors="pt")
        tt = self.teacher_tok([TeacherTokenizer.preprocess(s) for s in seqs], padding="max_length", max_length=L,
                              truncation=True, return_tensors="pt")
        return {"input_ids": st["input_ids"], "attention_mask": st["attention_mask"],
                "teacher_input_ids": tt["input_ids"], "teacher_attention_mask": tt["attention_mask"],
                # host-side row lengths: the teacher drops the padding before its first layer
                "teacher_lengths": tt["attention_mask"].sum(dim=1).tolist()}


def distillation_loss(student: ProtX, batch: dict, teacher=None) -> torch.Tensor:
    """sum over features, mean over real tokens of (student - teacher)^2."""
    ids, mask = batch["input_ids"], batch["attention_mask"]
    if "teacher_embeddings" in batch:
        target = batch["teacher_embeddings"]
    else:
        with torch.no_grad():
            target = teacher(batch["teacher_input_ids"], batch["teacher_attention_mask"],
                             lengths=batch.get("teacher_lengths"))
    out = student(ids, mask, training_mode=True)["last_hidden_state"]
    B, S, D = out.shape
    return ops.masked_mse(out.reshape(B * S, D), target.reshape(B * S, D).to(out.dtype), mask.reshape(-1))


REFERENCE_TRAINING_CONFIG_KEYS = (
    "train_fasta", "val_fasta", "train_h5_prefix", "val_h5_prefix", "num_epochs", "batch_size", "learning_rate",
    "gradient_accumulation_steps", "lr_scheduler", "lr_scheduler_kwargs", "max_seq_len", "max_seqs_num",
    "val_ratio", "on_the_fly", "sharded", "project_name")


def resolve_config_from_manifest(cfg: DistillationConfig) -> DistillationConfig:
    """Dataset location and geometry from `<dataset_dir>/.data_manifest`
    (reference: distillation/pipeline.py:149-340). Without a dataset directory the explicit paths of
    the configuration are used, which is how a run resumed through its `training_config.json`
    arrives (reference: cli/distill.py:406-425)."""
    if not cfg.dataset_dir:
        need = ("train_fasta", "val_fasta") if cfg.on_the_fly else ("train_h5_prefix", "val_h5_prefix")
        missing = [k for k in need if not getattr(cfg, k)]
        if missing or not cfg.max_seq_len:
            raise ValueError("dataset_dir is required unless " + ", ".join(need) + " and max_seq_len are given")
        if not cfg.train_sequences:
            if cfg.on_the_fly:
                from nanoplm_b200.data.fasta import count_fasta
                cfg.train_sequences, cfg.val_sequences = count_fasta(cfg.train_fasta), count_fasta(cfg.val_fasta)
            else:
                cfg.train_sequences = len(LoadKDDataset(cfg.train_h5_prefix))
                cfg.val_sequences = len(LoadKDDataset(cfg.val_h5_prefix))
        return cfg
    info = validate_distillation_dataset(cfg.dataset_dir)
    m: DistillationManifest = info["manifest"]
    paths = get_dataset_paths(cfg.dataset_dir, m)
    cfg.max_seq_len, cfg.on_the_fly = m.max_seq_len, m.on_the_fly
    cfg.train_sequences, cfg.val_sequences, cfg.val_ratio = m.train_sequences, m.val_sequences, m.val_ratio
    cfg.max_seqs_num = m.seqs_num
    if m.on_the_fly:
        cfg.train_fasta, cfg.val_fasta = str(paths["train_fasta"]), str(paths["val_fasta"])
    else:
        cfg.train_h5_prefix, cfg.val_h5_prefix = str(paths["train_h5_prefix"]), str(paths["val_h5_prefix"])
        cfg.sharded = bool(m.sharded)
    return cfg


def _save_student(engine: ShardedEngine, path: Path, write: bool) -> None:
    """Gathers the fp32 student weights (a collective: EVERY rank must call this) and writes them
    on the rank that passes write=True."""
    sd = {k: v.contiguous() for k, v in engine.full_state_dict_model().items()}
    if not write:
        return
    try:
        from safetensors.torch import save_file
        save_file(sd, str(path / "model.safetensors"))
    except ImportError:
        torch.save(sd, path / "pytorch_model.bin")


def run_distillation(model_config: StudentConfig, cfg: DistillationConfig,
                     resume_config: Optional[ResumeConfig] = None, teacher=None,
                     max_steps: Optional[int] = None) -> dict:
    set_seed(cfg.seed)
    cfg = resolve_config_from_manifest(cfg)
    device, rank, world, local_rank = init_distributed(cfg.multi_gpu)
    is_main, distributed = rank == 0, world > 1
    student = ProtX(model_config)
    use_bf16 = cfg.bf16 and device.type == "cuda"
    hyper = AdamWHyper(lr=float(cfg.learning_rate), weight_decay=0.01, max_grad_norm=float(cfg.max_grad_norm))
    engine = ShardedEngine(student, hyper, device, compute_dtype=torch.bfloat16 if use_bf16 else torch.float32,
                           fused_comm=bool(getattr(cfg, "fused_comm", True)), decay_all=True)
    student.train()
    if cfg.on_the_fly and teacher is None:
        from nanoplm_b200.models.teacher import T5EncoderTeacher
        if cfg.teacher_random_init:
            teacher = T5EncoderTeacher(cfg.teacher, random_init=True, seed=cfg.seed)
        else:
            teacher = T5EncoderTeacher.from_pretrained(cfg.teacher.name)
    if teacher is not None and hasattr(teacher, "encoder_model"):
        teacher = teacher.encoder_model             # a `ProtT5`-style wrapper (reference: teacher/base.py)
    if teacher is not None:
        teacher.to(device)
        if use_bf16:
            teacher.to(torch.bfloat16)

    collator = DistillDataCollator(cfg.on_the_fly, cfg.max_seq_len)
    if cfg.on_the_fly:
        train_ds = KDDatasetOnTheFly(cfg.train_fasta, cfg.max_seqs_num, rank, world)
        val_ds = KDDatasetOnTheFly(cfg.val_fasta, None, rank, world)
        train_loader = DataLoader(train_ds, batch_size=cfg.batch_size, collate_fn=collator, num_workers=0)
        val_loader = DataLoader(val_ds, batch_size=cfg.batch_size, collate_fn=collator, num_workers=0)
        # sequences are dealt round-robin, so ranks hold n // world or n // world + 1 of them: every
        # rank runs the same number of micro-batches (the surplus sequence of some ranks is dropped),
        # otherwise the ranks would disagree on the number of collective optimizer steps
        n_train = cfg.train_sequences if cfg.max_seqs_num is None else min(cfg.train_sequences, cfg.max_seqs_num)
        per_rank = n_train // world
        if per_rank == 0:
            raise ValueError(f"{n_train} training sequences cannot feed {world} ranks")
        sampler = None
    else:
        train_ds = LoadKDDataset(cfg.train_h5_prefix, cfg.max_open_files, cfg.chunk_size, cfg.prefetch_batches,
                                 cfg.use_threading, seed=cfg.seed)
        val_ds = LoadKDDataset(cfg.val_h5_prefix, cfg.max_open_files, cfg.chunk_size, cfg.prefetch_batches,
                               cfg.use_threading)
        # pads by wrapping around so every rank sees exactly ceil(n / world) samples
        sampler = ResumableDistributedSampler(len(train_ds), world, rank, True, cfg.seed)
        train_loader = DataLoader(train_ds, batch_size=cfg.batch_size, sampler=sampler, collate_fn=collator,
                                  num_workers=0, drop_last=False)
        val_loader = DataLoader(val_ds, batch_size=cfg.batch_size, collate_fn=collator, num_workers=0,
                                sampler=ResumableDistributedSampler(len(val_ds), world, rank, False, 0))
        per_rank = len(sampler)
    accum = max(1, cfg.gradient_accumulation_steps)
    micro_per_epoch = max(1, math.ceil(per_rank / cfg.batch_size))
    steps_per_epoch = max(1, math.ceil(micro_per_epoch / accum))

    resume = resume_config or ResumeConfig()
    samples_per_step = cfg.batch_size * accum * world
    plan = prepare_run_and_steps(cfg.ckp_dir, cfg.num_epochs, cfg.logging_steps, cfg.eval_steps, cfg.save_steps,
                                 resume.is_resume, resume.checkpoint_dir, resume.extra_epochs,
                                 cfg.train_sequences, samples_per_step, create=is_main)
    if distributed:
        holder = [plan]
        dist.broadcast_object_list(holder, src=0)
        plan = holder[0]
    total_steps = plan.num_epochs * steps_per_epoch
    warmup = math.ceil(total_steps * cfg.warmup_ratio) if cfg.warmup_ratio < 1 else int(cfg.warmup_ratio)
    sched = make_distill_schedule(cfg.lr_scheduler, hyper.lr, warmup, total_steps, **(cfg.lr_scheduler_kwargs or {}))
    out_dir = Path(plan.output_dir)
    global_step = 0
    if resume.is_resume:
        ck = Path(resume.checkpoint_dir)
        if (ck / "model.safetensors").exists():
            from safetensors.torch import load_file
            engine.load_model_state_dict(load_file(str(ck / "model.safetensors")))
        elif (ck / "pytorch_model.bin").exists():
            engine.load_model_state_dict(torch.load(ck / "pytorch_model.bin", map_location="cpu", weights_only=True))
        if (ck / "optimizer.pt").exists():
            engine.load_optimizer_state_dict(torch.load(ck / "optimizer.pt", map_location="cpu", weights_only=True))
        if (ck / "scheduler.pt").exists():
            sched.load_state_dict(torch.load(ck / "scheduler.pt", map_location="cpu", weights_only=False))
        if (ck / "trainer_state.json").exists():
            global_step = int(json.loads((ck / "trainer_state.json").read_text()).get("global_step", 0))
        logger.info(f"Resumed distillation at step {global_step}")
    if is_main:
        (out_dir / "training_config.json").write_text(json.dumps(
            # the reference's flat keys (distillation/pipeline.py:557-576) first, then the full sections
            {**{k: getattr(cfg, k) for k in REFERENCE_TRAINING_CONFIG_KEYS},
             "train_sequences": cfg.train_sequences, "val_sequences": cfg.val_sequences,
             "model": as_plain_dict(model_config), "distillation": as_plain_dict(cfg),
             "total_steps": total_steps, "warmup_steps": warmup}, indent=2, default=str), encoding="utf-8")
    sink = MetricsSink(str(out_dir), cfg.project_name, plan.wandb_run_name, as_plain_dict(cfg), is_main)
    heartbeat = watchdog = None
    if cfg.heartbeat_seconds and cfg.heartbeat_seconds > 0:      # same scheme as the pretraining pipeline
        from nanoplm_b200.runtime.watchdog import Heartbeat, Watchdog
        heartbeat = Heartbeat(out_dir / "heartbeat", rank, cfg.heartbeat_seconds).start()
        if is_main and distributed:
            stall = float(cfg.heartbeat_stall_seconds or 0)
            watchdog = Watchdog(out_dir / "heartbeat", world, max_age=6 * cfg.heartbeat_seconds + 30,
                                max_step_age=stall if stall > 0 else None, interval=cfg.heartbeat_seconds).start()

    def to_dev(b):
        return {k: (v.to(device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in b.items()}

    @torch.no_grad()
    def evaluate() -> float:
        student.eval()
        tot = torch.zeros(2, dtype=torch.float64, device=device)
        for b in val_loader:
            b = to_dev(b)
            tot[0] += distillation_loss(student, b, teacher).double() * b["input_ids"].shape[0]
            tot[1] += b["input_ids"].shape[0]
        if distributed:
            dist.all_reduce(tot)
        student.train()
        return float(tot[0] / tot[1].clamp(min=1))

    def check_device_status() -> None:
        if device.type == "cuda":
            from nanoplm_b200.ops import _lib
            _lib.check_status()

    def save(step: int) -> None:
        check_device_status()                      # never persist state after a failed kernel
        sd_opt = engine.optimizer_state_dict()     # collective
        d = out_dir / f"checkpoint-{step}"
        tmp = out_dir / f".tmp-checkpoint-{step}"
        if is_main:
            tmp.mkdir(parents=True, exist_ok=True)
        _save_student(engine, tmp, write=is_main)  # collective
        if is_main:
            torch.save(sd_opt, tmp / "optimizer.pt")
            torch.save(sched.state_dict(), tmp / "scheduler.pt")
            (tmp / "trainer_state.json").write_text(json.dumps({"global_step": step}), encoding="utf-8")
            if d.exists():
                import shutil
                shutil.rmtree(d)
            os.replace(tmp, d)
        if distributed:
            dist.barrier()

    losses, evals = [], []
    acc = torch.zeros((), device=device)
    win, win_n, t0, seen = torch.zeros((), device=device), 0, time.perf_counter(), 0
    start_epoch = global_step // steps_per_epoch
    # a checkpoint taken inside an epoch: skip the micro-batches that epoch already consumed
    skip_micro = (global_step % steps_per_epoch) * accum
    done = False
    for epoch in range(start_epoch, plan.num_epochs):
        if sampler is not None:
            sampler.set_epoch(epoch)
            if skip_micro:
                sampler.fast_forward(skip_micro * cfg.batch_size)   # O(1): the loader starts past them
        micro = skip_micro if sampler is not None else 0
        to_skip = 0 if sampler is not None else skip_micro          # iterable dataset: read and drop
        skip_micro = 0
        for b in train_loader:
            if to_skip:
                to_skip -= 1
                micro += 1
                continue
            b = to_dev(b)
            loss = distillation_loss(student, b, teacher)
            loss.backward()
            acc += loss.detach().float()
            seen += int(b["input_ids"].shape[0])
            micro += 1
            if micro % accum and micro != micro_per_epoch:
                continue
            n_acc = accum if micro % accum == 0 else micro % accum
            lr = sched.get_lr()
            gn = engine.step(lr, n_acc)
            sched.step()
            global_step += 1
            if heartbeat is not None:
                heartbeat.step = global_step
            if os.environ.get("NPLM_INJECT_FAULT"):     # host-side failure for recovery tests, between steps
                from nanoplm_b200.runtime.faults import maybe_inject
                maybe_inject(rank, global_step)
            win += acc / n_acc
            acc.zero_()
            win_n += 1
            if global_step % plan.logging_steps == 0:
                lv = float(win / max(1, win_n))
                check_device_status()
                dt = time.perf_counter() - t0
                losses.append((global_step, lv))
                sink.log({"train/global_step": global_step, "train/loss": lv, "train/grad_norm": float(gn),
                          "train/learning_rate": lr, "train/samples_per_sec": seen * world / max(dt, 1e-9)})
                if is_main:
                    logger.info(f"[step {global_step}/{total_steps}] loss={lv:.5f} lr={lr:.2e} grad_norm={float(gn):.4f}")
                win.zero_()
                win_n, t0, seen = 0, time.perf_counter(), 0
            if global_step % plan.eval_steps == 0:
                ev = evaluate()
                evals.append((global_step, ev))
                sink.log({"train/global_step": global_step, "eval/loss": ev})
                if is_main:
                    logger.info(f"[step {global_step}] eval_loss={ev:.5f}")
            if global_step % plan.save_steps == 0:
                save(global_step)
            if max_steps is not None and global_step >= max_steps:
                done = True
                break
            if micro >= micro_per_epoch:
                break     # every rank stops after the same number of micro-batches
        if done:
            break
    save(global_step)
    _save_student(engine, out_dir, write=is_main)   # collective: every rank takes part
    ev = evaluate()
    sink.log({"train/global_step": global_step, "eval/loss": ev})
    sink.finish(str(out_dir))
    if watchdog is not None:
        watchdog.stop()
    if heartbeat is not None:
        heartbeat.stop()
    check_device_status()
    logger.info("Distillation complete.")
    return {"output_dir": str(out_dir), "losses": losses, "eval_losses": evals + [(global_step, ev)],
            "global_step": global_step, "student": student, "engine": engine}
