"""Run directories, batch arithmetic and resume bookkeeping.

Layout and rules follow the reference (src/nanoplm/pretraining/utils.py:21-265):
`<ckp_dir>/run-DDMMHHMM[-k]/{run_name.txt,.resume_counter,checkpoint-<step>/,archived_<ts>/}`;
gradient accumulation is derived from the token budget; on resume the run continues in the
checkpoint's parent directory, checkpoints from "the future" are archived, and the W&B name gets a
`-re<k>` suffix.
"""
from __future__ import annotations

import math
import os
import shutil
from dataclasses import dataclass
from datetime import datetime
from pathlib import Path
from typing import Optional, Union

from nanoplm_b200.utils.logging import logger


@dataclass
class BatchSetup:
    grad_accum_steps: int
    global_batch_size_samples: int
    achieved_global_batch_tokens: int


def compute_batch_setup(global_batch_size: int, micro_batch_size: int, max_seq_len: int,
                        world_size: int) -> BatchSetup:
    if global_batch_size <= 0:
        raise ValueError(f"global_batch_size must be > 0, got {global_batch_size}")
    per_micro = micro_batch_size * max_seq_len * world_size
    if per_micro <= 0:
        raise ValueError(f"Invalid token throughput per micro-step: {per_micro}. Check "
                         "micro_batch_size, max_seq_len, and world_size.")
    accum = max(1, math.ceil(global_batch_size / per_micro))
    logger.info(f"Batch setup: target={global_batch_size:,} tok, micro_step={per_micro:,} tok, "
                f"grad_accum={accum}, achieved={accum * per_micro:,} tok")
    return BatchSetup(accum, accum * micro_batch_size * world_size, accum * per_micro)


def get_num_workers(user_value: Union[int, str], world_size: int) -> int:
    if isinstance(user_value, str) and user_value == "auto":
        cores = os.cpu_count() or 1
        return max(1, min(4 * max(1, world_size), max(1, cores - 2)))
    try:
        v = int(user_value)
    except (TypeError, ValueError):
        raise ValueError(f"Invalid num_workers value: {user_value}. Must be a non-negative integer or 'auto'")
    if v < 0:
        raise ValueError(f"Invalid num_workers value: {user_value}. Must be a non-negative integer")
    return v


def resolve_world_size(multi_gpu: bool, world_size: Union[int, str]) -> int:
    if not multi_gpu:
        return 1
    if "WORLD_SIZE" in os.environ:
        return int(os.environ["WORLD_SIZE"])
    if isinstance(world_size, str) and world_size == "auto":
        import torch
        return max(1, torch.cuda.device_count())
    return max(1, int(world_size))


def archive_future_checkpoints(run_dir: Path, resume_step: int) -> Optional[Path]:
    """Moves checkpoint-N with N > resume_step into archived_<timestamp>/ (kept, not deleted)."""
    future = []
    for d in Path(run_dir).glob("checkpoint-*"):
        try:
            step = int(d.name.split("-")[1])
        except (IndexError, ValueError):
            continue
        if step > resume_step:
            future.append((step, d))
    if not future:
        return None
    archive = Path(run_dir) / f"archived_{datetime.now().strftime('%Y%m%d_%H%M%S')}"
    archive.mkdir(exist_ok=True)
    for step, d in sorted(future):
        logger.info(f"Archiving checkpoint-{step} to {archive.name}/")
        shutil.move(str(d), str(archive / d.name))
    return archive


@dataclass
class RunPlan:
    run_name: str
    wandb_run_name: str
    output_dir: str
    num_epochs: int
    logging_steps: int
    eval_steps: int
    save_steps: int
    resume_step: Optional[int]


def prepare_run_and_steps(ckp_dir: str, num_epochs: int, logging_steps: int, eval_steps: int,
                          save_steps: int, resume_is: bool, resume_checkpoint_dir: str,
                          extra_epochs: Optional[int], train_samples: int,
                          global_batch_size_samples: int, create: bool = True) -> RunPlan:
    root = Path(ckp_dir)
    resume_step = None
    if resume_is:
        ckpt = Path(resume_checkpoint_dir)
        run_name = ckpt.parent.name
        run_root = root / run_name
        if create:
            run_root.mkdir(parents=True, exist_ok=True)
            counter_file = run_root / ".resume_counter"
            try:
                counter = int(counter_file.read_text().strip()) + 1 if counter_file.exists() else 1
            except ValueError:
                counter = 1
            counter_file.write_text(str(counter), encoding="utf-8")
        else:
            cf = run_root / ".resume_counter"
            counter = int(cf.read_text().strip()) if cf.exists() else 1
        wandb_name = f"{run_name}-re{counter}"
        try:
            resume_step = int(ckpt.name.split("-")[1])
            if create:
                archive_future_checkpoints(run_root, resume_step)
        except (IndexError, ValueError):
            logger.warning(f"Could not extract step number from checkpoint path: {ckpt.name}.")
        if extra_epochs:
            num_epochs = num_epochs + int(extra_epochs)
    else:
        base = f"run-{datetime.now().strftime('%d%m%H%M')}"
        run_name, k = base, 2
        while (root / run_name).exists():
            run_name = f"{base}-{k}"
            k += 1
        run_root = root / run_name
        wandb_name = run_name
    if create:
        run_root.mkdir(parents=True, exist_ok=True)
        try:
            (run_root / "run_name.txt").write_text(run_name, encoding="utf-8")
        except OSError:
            pass
    steps_per_epoch = (train_samples + global_batch_size_samples - 1) // max(1, global_batch_size_samples)
    total = max(1, num_epochs * steps_per_epoch)
    clamp = lambda v: max(1, min(total, int(v)))
    return RunPlan(run_name, wandb_name, str(run_root), num_epochs, clamp(logging_steps),
                   clamp(eval_steps), clamp(save_steps), resume_step)
