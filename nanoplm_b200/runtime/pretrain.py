"""MLM pretraining pipeline (`nanoplm pretrain from-yaml`).

Same user-visible behaviour as the reference's pure pipeline
(src/nanoplm/pretraining/pure_pipeline.py:334-927): manifest-driven datasets, packing or padding
collators, token-budget gradient accumulation, AdamW with linear warm-up / decay, gradient
clipping at 1.0, periodic logging / evaluation / checkpoints in the same layout, resume.

How it runs is different: one process per GPU; parameters, gradients and optimizer state are owned
by `ShardedEngine` (flat buffers, sharded AdamW, one reduce-scatter + all-gather per optimizer step
rather than per micro-step); the model executes this package's sm_100a kernels; the step never
reads a device value on the host (token counts come from the collator, loss and gradient norm are
read only at logging boundaries); resume fast-forwards the sampler instead of re-reading data.
"""
from __future__ import annotations

import gc
import math
import os
import random
import contextlib
import time
from pathlib import Path
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, Sampler

from nanoplm_b200.config.schema import PretrainingConfig, PureTorchConfig, ResumeConfig, as_plain_dict
from nanoplm_b200.data.collators import PackingCollator, ProtDataCollatorForLM
from nanoplm_b200.data.manifest import read_manifest, validate_manifest_for_pipeline
from nanoplm_b200.data.shards import ShardedDataset
from nanoplm_b200.models.encoder import ProtEncoderMLM, estimate_flops_per_token
from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
from nanoplm_b200.runtime import checkpoint as ckpt
from nanoplm_b200.runtime.metrics import MetricsSink
from nanoplm_b200.runtime.run_dirs import (compute_batch_setup, get_num_workers, prepare_run_and_steps,
                                           resolve_world_size)
from nanoplm_b200.parallel.muon import is_muon_optimizer
from nanoplm_b200.runtime.schedule import (WarmupLinearSchedule, get_warmup_steps,
                                           num_update_steps_per_epoch)
from nanoplm_b200.utils.logging import logger


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class ResumableDistributedSampler(Sampler):
    """Shuffled, rank-strided sampler with an O(1) fast-forward (`start_index`), so resuming in the
    middle of an epoch does not iterate over the data already consumed."""

    def __init__(self, n: int, world: int = 1, rank: int = 0, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False):
        self.n, self.world, self.rank, self.shuffle, self.seed = n, world, rank, shuffle, seed
        self.epoch, self.start_index = 0, 0
        self.per_rank = n // world if drop_last else math.ceil(n / world)
        self.drop_last = drop_last

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def fast_forward(self, samples: int) -> None:
        self.start_index = max(0, min(self.per_rank, samples))

    def __len__(self) -> int:
        return self.per_rank - self.start_index

    def __iter__(self):
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.n, generator=g).tolist()
        else:
            order = list(range(self.n))
        total = self.per_rank * self.world
        if not self.drop_last and total > len(order):
            order += order[: total - len(order)]
        mine = order[self.rank:total:self.world]
        start, self.start_index = self.start_index, 0
        return iter(mine[start:])


def init_distributed(multi_gpu: bool) -> tuple[torch.device, int, int, int]:
    """Returns (device, rank, world, local_rank); joins the process group when launched by torchrun."""
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    want = multi_gpu and int(os.environ.get("WORLD_SIZE", "1")) > 1
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
        device = torch.device(f"cuda:{local_rank}")
    else:
        device = torch.device("cpu")
    if want and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device.type == "cuda":
            dist.init_process_group(backend="nccl", device_id=device)
        else:
            dist.init_process_group(backend="gloo")
    if dist.is_initialized():
        return device, dist.get_rank(), dist.get_world_size(), local_rank
    return device, 0, 1, local_rank


def move_batch(batch: dict, device: torch.device) -> dict:
    out = {}
    for k, v in batch.items():
        if torch.is_tensor(v):
            if device.type == "cuda" and not v.is_pinned():
                v = v.pin_memory()
            out[k] = v.to(device, non_blocking=True)
        else:
            out[k] = v
    return out


def model_inputs(batch: dict) -> dict:
    keys = ("input_ids", "attention_mask", "labels", "cu_seqlens", "max_seqlen", "position_ids",
            "masked_idx", "masked_labels", "num_real_tokens")
    return {k: batch[k] for k in keys if k in batch}


def batch_token_counts(batch: dict) -> tuple[int, int]:
    """(real tokens, tokens including padding), from host-side values only."""
    ids = batch["input_ids"]
    if "num_real_tokens" in batch:
        return int(batch["num_real_tokens"]), int(ids.numel())
    if "attention_mask" in batch and not batch["attention_mask"].is_cuda:
        return int(batch["attention_mask"].sum()), int(ids.numel())
    if "cu_seqlens" in batch and not batch["cu_seqlens"].is_cuda:
        return int(batch["cu_seqlens"][-1]), int(ids.numel())
    return int(ids.numel()), int(ids.numel())


@torch.no_grad()
def evaluate(model, loader, device, distributed: bool) -> float:
    model.eval()
    total = torch.zeros(2, dtype=torch.float64, device=device)
    for batch in loader:
        rows = batch["input_ids"].size(0)
        out = model(**model_inputs(move_batch(batch, device)))
        total[0] += out["loss"].double() * rows
        total[1] += rows
    if distributed:
        dist.all_reduce(total)
    model.train()
    return float(total[0] / total[1].clamp(min=1))


def build_collators(tokenizer, cfg: PretrainingConfig, pt: PureTorchConfig, max_seq_len: int, seed: int):
    kw = dict(mlm_probability=cfg.mlm_probability, mask_token_probability=cfg.mask_replace_prob,
              random_token_probability=cfg.random_token_prob, keep_probability=cfg.keep_probability)
    if pt.use_packing:
        train = PackingCollator(tokenizer, max_seq_len, **kw, target_rows=pt.target_packed_rows,
                                batch_size=cfg.micro_batch_size if pt.target_packed_rows else None, seed=seed)
    else:
        train = ProtDataCollatorForLM(tokenizer, **kw, seed=seed)
    return train, ProtDataCollatorForLM(tokenizer, **kw, seed=seed + 1)


def run_pretraining(model: ProtEncoderMLM, pretrain_config: PretrainingConfig,
                    pure_torch_config: Optional[PureTorchConfig] = None,
                    resume_config: Optional[ResumeConfig] = None, max_steps: Optional[int] = None,
                    on_step=None, final_checkpoint: bool = True) -> dict:
    """on_step: optional callable invoked after every optimizer step with a dict (global_step, this
    rank's real / raw token counts of the step, bytes copied host -> device and read back device ->
    host during the step); benchmarks time the loop with it. final_checkpoint=False skips the
    checkpoint at the end of the run."""
    cfg = pretrain_config
    pt = pure_torch_config or PureTorchConfig()
    os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")
    set_seed(cfg.seed)
    tokenizer = model.tokenizer
    dataset_dir = Path(cfg.dataset_dir)
    manifest = read_manifest(dataset_dir)
    validate_manifest_for_pipeline(manifest, "pretrain")
    train_dir, val_dir = dataset_dir / manifest.train_dir, dataset_dir / manifest.val_dir
    for d, what in ((train_dir, "Train"), (val_dir, "Validation")):
        if not d.exists():
            raise FileNotFoundError(f"{what} shard directory not found: {d}")
    train_ds, val_ds = ShardedDataset(train_dir), ShardedDataset(val_dir)
    logger.info(f"Loaded config from manifest: {dataset_dir} (max_length={manifest.max_seq_len}, "
                f"train={manifest.train_sequences}, val={manifest.val_sequences})")

    world_cfg = resolve_world_size(cfg.multi_gpu, cfg.world_size)
    device, rank, world, local_rank = init_distributed(cfg.multi_gpu)
    distributed = world > 1
    is_main = rank == 0
    batch = compute_batch_setup(cfg.global_batch_size, cfg.micro_batch_size, manifest.max_seq_len, world)
    grad_accum = batch.grad_accum_steps

    resume = resume_config or ResumeConfig()
    if is_main:
        plan = prepare_run_and_steps(cfg.ckp_dir, cfg.num_epochs, cfg.logging_steps, cfg.eval_steps,
                                     cfg.save_steps, resume.is_resume, resume.checkpoint_dir,
                                     resume.extra_epochs, manifest.train_sequences,
                                     batch.global_batch_size_samples)
        plans = [plan]
    else:
        plans = [None]
    if distributed:
        dist.broadcast_object_list(plans, src=0)
    plan = plans[0]
    output_dir, num_epochs = plan.output_dir, plan.num_epochs

    use_bf16 = cfg.bf16 and device.type == "cuda"
    hyper = AdamWHyper(lr=float(cfg.adam_learning_rate), beta1=float(cfg.adam_beta1),
                       beta2=float(cfg.adam_beta2), eps=float(cfg.adam_epsilon),
                       weight_decay=float(cfg.adam_weight_decay), max_grad_norm=float(cfg.max_grad_norm))
    opt_name = str(cfg.optimizer).lower()
    ep_size = int(getattr(cfg, "expert_parallel_size", 1) or 1)
    if ep_size > 1:
        # experts split over the data-parallel ranks (peer-memory dispatch / combine on CUDA)
        if ep_size > world or world % ep_size:
            raise ValueError(f"expert_parallel_size ({ep_size}) must divide the number of ranks ({world}): "
                             "the ranks form world / size groups, each holding every expert once")
        if opt_name not in ("adamw", "stable_adamw"):
            raise ValueError("expert parallelism is implemented for the AdamW engine only")
        from nanoplm_b200.parallel.expert_engine import (ExpertParallelEngine, make_expert_groups,
                                                         shard_model_experts)
        ep_group, edp_group = make_expert_groups(ep_size)
        if shard_model_experts(model, ep_group) == 0:
            raise ValueError("expert_parallel_size > 1 needs a model with model.moe configured")
        engine = ExpertParallelEngine(model, hyper, device,
                                      compute_dtype=torch.bfloat16 if use_bf16 else torch.float32,
                                      fused_comm=bool(cfg.fused_comm), ep_group=ep_group, edp_group=edp_group)
    elif opt_name in ("muon", "normuon"):
        from nanoplm_b200.parallel.muon import MuonEngine
        engine = MuonEngine(model, hyper, cfg, device)
    elif opt_name in ("adamw", "stable_adamw"):
        engine_cls = ShardedEngine
        if bool(getattr(cfg, "shard_params", False)) and distributed:
            # parameters, gradients' reduction and optimizer state split by row blocks; the all-gather
            # of the weights runs inside the forward GEMMs (reference: FSDP2, pure_pipeline.py:479-506)
            from nanoplm_b200.parallel.param_sharded import ParamShardedEngine
            engine_cls = ParamShardedEngine
        engine = engine_cls(model, hyper, device,
                            compute_dtype=torch.bfloat16 if use_bf16 else torch.float32,
                            fused_comm=bool(cfg.fused_comm))
    else:
        raise ValueError(f"Invalid optimizer: {cfg.optimizer}. Supported: [adamw, stable_adamw, muon, normuon]")
    model.train()
    # logging statistics: one kernel over peer memory instead of library all-reduces, where the
    # ranks can map each other's memory (same switch as the fused optimizer step)
    peer_stats = None
    if distributed and device.type == "cuda" and bool(cfg.fused_comm):
        from nanoplm_b200.comm.peer_stats import PeerStats
        peer_stats = PeerStats.try_create(device)
    if getattr(cfg, "fp8", False):
        if str(getattr(cfg, "fp8_recipe", "block128")) != "block128":
            raise ValueError(f"Unknown fp8_recipe {cfg.fp8_recipe!r}; supported: block128")
        from nanoplm_b200.ops import functional as _ops
        _ops.set_fp8(device.type == "cuda" and use_bf16)
        logger.info("FP8 (e4m3, block128) linear layers enabled")

    train_collator, eval_collator = build_collators(tokenizer, cfg, pt, manifest.max_seq_len,
                                                    cfg.seed + 1000 * rank)
    static_packing = pt.use_packing and pt.target_packed_rows is not None
    # optional: corrupt the batch on the GPU (Philox, keyed by seed / rank / micro-step) instead of
    # in the collator workers; the collator then only packs
    device_masking = bool(cfg.device_masking) and device.type == "cuda" and static_packing
    if device_masking:
        train_collator.masker.mlm_probability = 0.0
        mask_pool = torch.tensor(train_collator.masker.allowed_random_token_ids.tolist(), dtype=torch.int32,
                                 device=device)
        mask_micro = 0
    eval_sampler = ResumableDistributedSampler(len(val_ds), world, rank, False, cfg.seed)
    workers = get_num_workers(cfg.num_workers, world)
    loader_kw = dict(num_workers=workers, pin_memory=device.type == "cuda",
                     persistent_workers=workers > 0,
                     prefetch_factor=cfg.prefetch_factor if workers > 0 else None)
    # several ranks on packed batches: every optimizer step's sequences are dealt to the
    # (rank, micro-step) bins by cost, so no rank waits for another at the step's collective
    balanced = (bool(getattr(cfg, "balance_ranks", True)) and distributed and static_packing
                and len(train_ds) >= cfg.micro_batch_size * grad_accum * world)
    if balanced:
        from nanoplm_b200.data.sampler import BalancedBatchSampler
        train_sampler = BalancedBatchSampler(train_ds.sequence_lengths(), cfg.micro_batch_size, grad_accum, world,
                                             rank, True, cfg.seed, float(cfg.balance_quadratic),
                                             max_length=manifest.max_seq_len)
        train_loader = DataLoader(train_ds, batch_sampler=train_sampler, collate_fn=train_collator, **loader_kw)
        loader_len = len(train_sampler)
    else:
        train_sampler = ResumableDistributedSampler(len(train_ds), world, rank, True, cfg.seed)
        train_loader = DataLoader(train_ds, sampler=train_sampler, batch_size=cfg.micro_batch_size,
                                  collate_fn=train_collator, drop_last=static_packing, **loader_kw)
        loader_len = (len(train_sampler) // cfg.micro_batch_size if static_packing
                      else math.ceil(len(train_sampler) / cfg.micro_batch_size))
    eval_loader = DataLoader(val_ds, sampler=eval_sampler, batch_size=cfg.micro_batch_size,
                             collate_fn=eval_collator, drop_last=False, **loader_kw)
    steps_per_epoch = num_update_steps_per_epoch(loader_len, grad_accum)
    total_steps = num_epochs * steps_per_epoch
    warmup_steps = get_warmup_steps(total_steps, float(cfg.warmup_ratio))
    scheduler = WarmupLinearSchedule(hyper.lr, warmup_steps, total_steps)

    start_step = start_epoch = 0
    resume_micro = 0
    if resume.is_resume:
        logger.info(f"Resuming from checkpoint: {resume.checkpoint_dir}")
        start_step, start_epoch = ckpt.load_checkpoint(engine, scheduler, resume.checkpoint_dir)
        steps_done = max(0, start_step - start_epoch * steps_per_epoch)
        resume_micro = steps_done * grad_accum
        if resume_micro >= loader_len:
            resume_micro, start_epoch = 0, min(start_epoch + 1, num_epochs)
        logger.info(f"Resumed at global_step={start_step}, epoch={start_epoch}")

    sink = MetricsSink(output_dir, cfg.project_name, plan.wandb_run_name,
                       {"pretrain": as_plain_dict(cfg), "total_steps": total_steps, "warmup_steps": warmup_steps},
                       is_main, jsonl=cfg.metrics_jsonl)
    flops_per_token = estimate_flops_per_token(model.config, manifest.max_seq_len)
    heartbeat = watchdog = None
    if cfg.heartbeat_seconds and cfg.heartbeat_seconds > 0:
        from nanoplm_b200.runtime.watchdog import Heartbeat, Watchdog
        heartbeat = Heartbeat(Path(output_dir) / "heartbeat", rank, cfg.heartbeat_seconds).start()
        if is_main and distributed:
            # a rank that died stops beating; a rank stuck in a collective keeps beating but its
            # step stops advancing: both end the job instead of leaving it hung
            stall = float(getattr(cfg, "heartbeat_stall_seconds", 0) or 0)
            watchdog = Watchdog(Path(output_dir) / "heartbeat", world, max_age=6 * cfg.heartbeat_seconds + 30,
                                max_step_age=stall if stall > 0 else None,
                                interval=cfg.heartbeat_seconds).start()

    def check_device_status() -> None:
        """Bounded waits that ran out, peer time-outs and MoE capacity overflow set a device status
        word; training must not continue (and no checkpoint may be written) after that."""
        if device.type == "cuda":
            from nanoplm_b200.ops import _lib
            _lib.check_status()

    logger.info(f"Starting training: epochs={num_epochs}, total_steps={total_steps}, "
                f"warmup_steps={warmup_steps}, grad_accum={grad_accum}, world={world}, "
                f"params={engine.num_parameters():,}, bf16={use_bf16}")

    moe_layers = [m for m in model.modules() if hasattr(m, "dropped_rows") and hasattr(m, "experts_Wi")]
    use_nvtx = bool(getattr(cfg, "nvtx_ranges", False)) and device.type == "cuda"
    if device.type == "cuda":
        from nanoplm_b200.ops import kernels as _kernels
        _kernels.set_attention_deterministic(bool(getattr(cfg, "deterministic_attention", False)))

    def _range(name: str):
        """NVTX range (`pretraining.nvtx_ranges: true`) so that a timeline profiler shows the phases
        of a step; a no-op context otherwise."""
        return torch.cuda.nvtx.range(name) if use_nvtx else contextlib.nullcontext()

    global_step = start_step
    window_loss = torch.zeros((), dtype=torch.float32, device=device)
    accum_loss = torch.zeros((), dtype=torch.float32, device=device)
    window_steps = 0
    tok = raw_tok = 0
    t0: Optional[float] = None
    last_grad_norm = None
    first = True
    result = {"output_dir": output_dir, "losses": [], "eval_losses": []}
    done = False
    step_tok = step_raw = step_h2d = 0

    for epoch in range(start_epoch, num_epochs):
        train_sampler.set_epoch(epoch)
        offset = 0
        if resume_micro > 0 and epoch == start_epoch:
            train_sampler.fast_forward(resume_micro if balanced else resume_micro * cfg.micro_batch_size)
            offset = resume_micro
            resume_micro = 0
        n_micro = offset + len(train_loader)
        for i, host_batch in enumerate(train_loader):
            micro_step = offset + i
            if t0 is None:
                t0 = time.perf_counter()
            a, b = batch_token_counts(host_batch)
            tok += a
            raw_tok += b
            step_tok += a
            step_raw += b
            step_h2d += sum(v.numel() * v.element_size() for v in host_batch.values() if torch.is_tensor(v))
            dev_batch = move_batch(host_batch, device)
            if device_masking:
                from nanoplm_b200.ops import kernels as K
                mk = train_collator.masker
                ids_m, lab_m = K.mlm_mask(dev_batch["input_ids"], a, tokenizer.all_special_ids, mk.mask_token_id,
                                          mask_pool, float(cfg.mlm_probability), mk.p_mask, mk.p_rand,
                                          cfg.seed * 1000003 + rank, mask_micro)
                mask_micro += 1
                dev_batch.update(input_ids=ids_m, labels=lab_m)
                dev_batch.pop("masked_idx", None)
                dev_batch.pop("masked_labels", None)
            boundary = (micro_step + 1) % grad_accum == 0 or micro_step + 1 == n_micro
            if boundary and hasattr(engine, "begin_last_microstep"):
                engine.begin_last_microstep()    # gradient reduction overlaps this backward pass
            with _range("forward"):
                out = model(**model_inputs(dev_batch))
                loss = out["loss"]
            with _range("backward"):
                loss.backward()
            accum_loss += loss.detach().float()
            if not boundary:
                continue
            n_acc = (micro_step % grad_accum) + 1
            lr = scheduler.get_lr()
            with _range("optimizer_step"):
                last_grad_norm = engine.step(lr, n_acc)
            scheduler.step()
            global_step += 1
            if heartbeat is not None:
                heartbeat.step = global_step
            if os.environ.get("NPLM_INJECT_FAULT"):     # host-side failure for recovery tests, between steps
                from nanoplm_b200.runtime.faults import maybe_inject
                maybe_inject(rank, global_step)
            window_loss += accum_loss / n_acc
            accum_loss.zero_()
            window_steps += 1

            if global_step % plan.logging_steps == 0:
                if device.type == "cuda":
                    torch.cuda.synchronize()
                check_device_status()     # the loop synchronises here anyway
                elapsed = time.perf_counter() - t0
                stats = torch.tensor([tok, raw_tok, elapsed], dtype=torch.float64, device=device)
                if peer_stats is not None:
                    stats = torch.tensor(peer_stats.all_reduce([tok, raw_tok, elapsed], max_mask=0b100),
                                         dtype=torch.float64)
                elif distributed:
                    mx = stats[2:].clone()
                    dist.all_reduce(stats[:2])
                    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                    stats[2] = mx[0]
                tps, raw_tps = float(stats[0] / stats[2]), float(stats[1] / stats[2])
                h100, b200 = sink.mfu(raw_tps, flops_per_token, world)
                loss_val = float(window_loss / max(1, window_steps))
                gn = float(last_grad_norm)
                result["losses"].append((global_step, loss_val))
                payload = {"train/global_step": global_step, "train/loss": loss_val,
                           "train/grad_norm": gn, "train/learning_rate": lr, "train/adamw_lr": lr,
                           "train/epoch": epoch + (micro_step + 1) / max(1, n_micro),
                           "train/tokens_per_sec": tps, "train/raw_tokens_per_sec": raw_tps,
                           "train/h100_mfu": h100, "train/b200_mfu": b200,
                           "train/step_ms_max_rank": 1e3 * float(stats[2]) / max(1, window_steps)}
                # Muon / NorMuon: the matrices' rate, which follows the same schedule from its own base
                # value (reference: pure_pipeline.py:766-772, 825-827)
                muon_lr = float(engine.muon_lr) if is_muon_optimizer(engine) else None
                if muon_lr is not None:
                    payload["train/muon_lr"] = muon_lr
                if moe_layers:      # rows dropped by full expert buffers (skewed routing), this rank, so far
                    payload["train/moe_dropped_rows"] = sum(m.dropped_rows() for m in moe_layers)
                sink.log(payload)
                if is_main:
                    logger.info(f"[step {global_step}/{total_steps}] loss={loss_val:.4f} lr={lr:.2e} "
                                + (f"muon_lr={muon_lr:.2e} " if muon_lr is not None else "") +
                                f"grad_norm={gn:.4f} tok/s={tps:,.0f} raw_tok/s={raw_tps:,.0f} "
                                f"h100_mfu={h100:.2%} b200_mfu={b200:.2%}")
                window_loss.zero_()
                window_steps, tok, raw_tok, t0 = 0, 0, 0, None
                step_d2h = 8          # window loss + gradient norm read back as two fp32 scalars
            else:
                step_d2h = 0
            if on_step is not None:
                on_step({"global_step": global_step, "tokens": step_tok, "raw_tokens": step_raw,
                         "h2d_bytes": step_h2d, "d2h_bytes": step_d2h})
            step_tok = step_raw = step_h2d = 0

            if first:  # keep the collector away from the step loop (reference: pure_pipeline.py:843-853)
                first = False
                gc.collect()
                gc.freeze()
                gc.disable()
            elif global_step % 5000 == 0:
                gc.collect()

            if global_step % plan.eval_steps == 0:
                ev = evaluate(model, eval_loader, device, distributed)
                result["eval_losses"].append((global_step, ev))
                sink.log({"train/global_step": global_step, "eval/loss": ev})
                if is_main:
                    logger.info(f"[step {global_step}] eval_loss={ev:.4f}")
            if global_step % plan.save_steps == 0:
                check_device_status()     # raises before a corrupted state could be persisted
                ckpt.save_checkpoint(engine, scheduler, global_step, epoch, output_dir, plan.logging_steps,
                                     plan.eval_steps, plan.save_steps, is_main, cfg.sharded_checkpoint,
                                     hf_files=bool(getattr(cfg, "hf_checkpoint_files", False)))
            if max_steps is not None and global_step - start_step >= max_steps:
                done = True
                break
        if done:
            break

    gc.enable()
    check_device_status()
    if distributed:
        dist.barrier()
    if final_checkpoint:
        ckpt.save_checkpoint(engine, scheduler, global_step, num_epochs, output_dir, plan.logging_steps,
                             plan.eval_steps, plan.save_steps, is_main, cfg.sharded_checkpoint,
                             hf_files=bool(getattr(cfg, "hf_checkpoint_files", False)))
    sink.finish(output_dir)
    if watchdog is not None:
        watchdog.stop()
    if heartbeat is not None:
        heartbeat.stop()
    check_device_status()
    logger.info("Pretraining complete.")
    result["global_step"] = global_step
    result["engine"] = engine
    return result


class TrainStep:
    """One optimizer step over a list of micro-batches: the programmatic training API.

        stepper = TrainStep(model, engine, scheduler, device)
        loss = stepper.step_from_host(host_batches)   # pinned host tensors in, python float out

    `step_from_host` copies every micro-batch host->device, runs forward/backward, applies the
    optimizer step and reads the mean loss back (one device->host copy per step).
    `step_on_device` does the same for batches that already live on the GPU and returns the loss as
    a device tensor without synchronising.
    """

    def __init__(self, model, engine, scheduler, device):
        self.model, self.engine, self.scheduler, self.device = model, engine, scheduler, torch.device(device)
        self._acc = torch.zeros((), dtype=torch.float32, device=self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # host->device copies run on their own stream, one micro-batch ahead of the compute stream
        self._copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def _prefetch(self, b: dict):
        """Starts the host->device copy of one micro-batch; returns (device batch, ready event)."""
        self.h2d_bytes += sum(v.numel() * v.element_size() for v in b.values() if torch.is_tensor(v))
        if self._copy_stream is None:
            return move_batch(b, self.device), None
        with torch.cuda.stream(self._copy_stream):
            moved = move_batch(b, self.device)
            ready = torch.cuda.Event()
            ready.record(self._copy_stream)
        return moved, ready

    def _run(self, batches, from_host: bool) -> torch.Tensor:
        self._acc.zero_()
        pending = self._prefetch(batches[0]) if (from_host and batches) else None
        for i, b in enumerate(batches):
            if from_host:
                b, ready = pending
                pending = self._prefetch(batches[i + 1]) if i + 1 < len(batches) else None
                if ready is not None:
                    cur = torch.cuda.current_stream(self.device)
                    cur.wait_event(ready)
                    for v in b.values():
                        if torch.is_tensor(v):
                            v.record_stream(cur)     # allocated on the copy stream, used on this one
            if i + 1 == len(batches) and hasattr(self.engine, "begin_last_microstep"):
                self.engine.begin_last_microstep()   # gradient reduction overlaps the last backward pass
            out = self.model(**model_inputs(b))
            out["loss"].backward()
            self._acc += out["loss"].detach().float()
        self.engine.step(self.scheduler.get_lr(), len(batches))
        self.scheduler.step()
        return self._acc / max(1, len(batches))

    def step_on_device(self, dev_batches) -> torch.Tensor:
        return self._run(dev_batches, False)

    def step_from_host(self, host_batches) -> float:
        loss = self._run(host_batches, True)
        self.d2h_bytes += loss.element_size()
        return float(loss.item())


# The reference has two entry points, the HF-Trainer pipeline `run_pretraining`
# (src/nanoplm/pretraining/pipeline.py:107-295) and `run_pure_pretraining`
# (src/nanoplm/pretraining/pure_pipeline.py:334-927); both names lead to the one native pipeline.
run_pure_pretraining = run_pretraining
