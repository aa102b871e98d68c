"""Training metrics: console line, JSONL file, optional Weights & Biases.

Metric keys follow the reference (pure_pipeline.py:815-841): train/{global_step, loss, grad_norm,
learning_rate, adamw_lr, epoch, tokens_per_sec, raw_tokens_per_sec, h100_mfu} and eval/loss, plus
train/b200_mfu (against the measured cuBLAS bf16 throughput of this GPU pool) and
train/step_ms_max_rank. W&B failures never stop training; the JSONL file works offline.
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Optional

from nanoplm_b200.utils.logging import logger
from nanoplm_b200.utils.peaks import measured_peaks

H100_PEAK_TFLOPS = 989.4  # the constant the reference reports MFU against (pure_pipeline.py:79-80)


class MetricsSink:
    def __init__(self, output_dir: str, project: str, run_name: str, config: dict, is_main: bool,
                 jsonl: bool = True, use_wandb: Optional[bool] = None):
        self.is_main = is_main
        self.jsonl_path = Path(output_dir) / "metrics.jsonl" if (jsonl and is_main) else None
        self.wandb = None
        self.b200_peak = measured_peaks().get("bf16_tflops_sustained", 1323.0)
        if use_wandb is None:
            use_wandb = os.environ.get("WANDB_MODE", "").lower() not in ("disabled", "offline-none")
        if is_main and use_wandb:
            try:
                import wandb
                wandb.init(project=project, name=run_name, config=config)
                if wandb.run is not None:
                    wandb.define_metric("train/global_step")
                    wandb.define_metric("*", step_metric="train/global_step", step_sync=True)
                    self.wandb = wandb
            except Exception as exc:
                logger.warning(f"W&B init failed, continuing without logging. Error: {exc}")

    def log(self, payload: dict) -> None:
        if not self.is_main:
            return
        if self.jsonl_path is not None:
            with open(self.jsonl_path, "a", encoding="utf-8") as f:
                f.write(json.dumps({"time": time.time(), **payload}) + "\n")
        if self.wandb is not None:
            try:
                self.wandb.log(payload)
            except Exception as exc:
                logger.warning(f"W&B log failed; disabling logging. Error: {exc}")
                self.wandb = None

    def mfu(self, raw_tokens_per_sec: float, flops_per_token: int, world: int) -> tuple[float, float]:
        per_gpu = raw_tokens_per_sec * flops_per_token / max(1, world)
        return per_gpu / (H100_PEAK_TFLOPS * 1e12), per_gpu / (self.b200_peak * 1e12)

    def finish(self, output_dir: str) -> None:
        if self.wandb is not None and self.is_main:
            try:
                (Path(output_dir) / "wandb_run_id.txt").write_text(self.wandb.run.id, encoding="utf-8")
                self.wandb.finish()
            except Exception as exc:
                logger.warning(f"W&B finalize failed. Error: {exc}")
