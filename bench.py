"""Headline benchmark: MLM pretraining tokens/sec of the default 1024x16 encoder (bf16, sequence-
packed varlen batches of 65 536 flat tokens per GPU per micro-batch, 2^20 flat tokens per optimizer
step over all GPUs, AdamW + gradient clipping), on synthetic protein data with random-init weights.

    python bench.py --gpus N --steps K --warmup W [--impl own|reference]

N > 1 is launched as `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...`.
Rank 0 prints ONE JSON line. `value` = real (non-padding) tokens per second over all GPUs for K
optimizer steps, timed on the device with CUDA events between barrier + synchronize pairs, maximum
over ranks. `e2e` is the same metric through the user-facing pipeline
(`nanoplm_b200.runtime.pretrain.run_pretraining` on a shard dataset: DataLoader workers, packing
collator, every micro-batch copied from pinned host memory, loss read back every step).
`no_trim_value` repeats the device-timed measurement over the full static shape (padding tail left
in place), `exposed_comm_ms` is the part of the optimizer step's communication that is not hidden
under the backward pass, `step_ms` the spread of the timed steps.

`--impl reference` runs the unmodified reference package installed under baseline/_ref through its
own `run_pure_pretraining` (FSDP2 / torch.compile / flash-attn path) on the same synthetic data and
batch geometry; the only instrumentation is a wrapper around `torch.optim.AdamW.step` that records
CUDA events at the boundaries of the timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
# both arms: same allocator policy as the reference's own pipeline sets for itself
os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")

MODEL = dict(hidden_size=1024, intermediate_size=2048, num_hidden_layers=16, num_attention_heads=16,
             vocab_size=32, max_position_embeddings=1024)
MAX_SEQ_LEN = 512            # tokens per sequence including </s>; lengths uniform in [20, 512]
MIN_SEQ_LEN = 20
TARGET_ROWS = 128            # 128 rows x 512 = 65 536 flat tokens per micro-batch per GPU
SEQS_PER_MICRO = 208         # mean 55.3 K real tokens; 4.5 sigma below the 128-row capacity
MICRO_PER_STEP = 16          # 16 x 65 536 = 2^20 flat tokens per optimizer step (all GPUs together)
MLM_PROB = 0.15
BASELINE_VALUE = None        # the reference publishes no throughput number


# ----------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.samples, self._t, self._p = gpu_index, [], None, None
        self._t0 = self._t1 = None

    def _run(self):
        for line in self._p.stdout:
            line = line.strip()
            if line:
                self.samples.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def start(self):
        """Starts ONE nvidia-smi process that prints a sample every 200 ms (a new process per sample would
        initialise NVML, and take the driver's locks, five times a second next to the launch thread).
        Call before the warm-up steps; only samples between begin() and stop() are used."""
        try:
            self._p = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                        "--format=csv,noheader,nounits", "-lms", "200"],
                                       stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._p = None
            return
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def begin(self):
        self._t0 = time.monotonic()

    def stop(self) -> dict:
        self._t1 = time.monotonic()
        if self._p is not None:
            self._p.terminate()          # our own child, by handle
            try:
                self._p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._p.kill()
        if self._t is not None:
            self._t.join(timeout=6)
        t0 = self._t0 if self._t0 is not None else 0.0
        rows = [f for (t, f) in self.samples if t0 <= t <= self._t1]
        sm, mx, reasons = [], 0.0, set()
        for s in rows:
            try:
                sm.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------- data
def make_sequences(n: int, seed: int):
    """uint8 token arrays (residues + </s>), total length uniform in [MIN_SEQ_LEN, MAX_SEQ_LEN]."""
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    return synthetic_token_sequences(n, MIN_SEQ_LEN - 1, MAX_SEQ_LEN - 1, seed)


def write_shard_dataset(out_dir: Path, n_train: int, n_val: int, seed: int) -> int:
    """Writes the dataset in the shard + manifest format both frameworks read; returns the number of
    real training tokens."""
    import numpy as np
    from nanoplm_b200.data.manifest import PretrainManifest, write_manifest
    total = 0
    for split, n, s in (("train", n_train, seed), ("val", n_val, seed + 1)):
        d = out_dir / split
        d.mkdir(parents=True, exist_ok=True)
        seqs = make_sequences(n, s)
        if split == "train":
            total = int(sum(len(x) for x in seqs))
        np.concatenate(seqs).astype(np.uint8).tofile(d / "shard_0000.bin")
        np.save(d / "shard_0000.idx.npy", np.asarray([len(x) for x in seqs], dtype=np.int32))
    write_manifest(out_dir, PretrainManifest(
        pipeline_mode="pretrain", seqs_num=n_train + n_val, min_seq_len=MIN_SEQ_LEN, max_seq_len=MAX_SEQ_LEN,
        val_ratio=n_val / (n_train + n_val), train_dir="train", val_dir="val", train_sequences=n_train,
        val_sequences=n_val, sharded=True, samples_per_shard=max(n_train, n_val)))
    return total


def config_block(n_gpus: int, accum: int) -> dict:
    return {"model": "nanoPLM default encoder: hidden 1024, intermediate 2048, 16 layers, 16 heads, "
                     "vocab 32, SwiGLU, RoPE, global/local(+-64) attention, 168.9 M parameters",
            "global_batch": MICRO_PER_STEP * TARGET_ROWS * MAX_SEQ_LEN, "seq_len": MAX_SEQ_LEN,
            "micro_batch_flat_tokens": TARGET_ROWS * MAX_SEQ_LEN, "sequences_per_micro_batch": SEQS_PER_MICRO,
            "grad_accum": accum, "parallelism": f"dp{n_gpus}" + ("-sharded-optimizer" if n_gpus > 1 else ""),
            "optimizer": "adamw lr 1e-3, clip 1.0", "mlm_probability": MLM_PROB,
            "tokens_counted": "real (non-padding) tokens; the flat batch also holds the padding tail",
            "l2_policy": "inputs larger than L2: every layer streams >= 128 MB of activations per micro-batch",
            "padding_tail": "both arms receive the same 65 536-token flat micro-batches (about 55.3 K real "
                            "tokens + padding tail); the own arm cuts the tail off on the host-known real-token "
                            "count before its first kernel (loss and gradients unchanged; --no-trim disables it), "
                            "the reference computes over the full static shape its compiler needs"}


# ----------------------------------------------------------------------------------- own arm
def _step_batches(step: int, rank: int, world: int, accum: int, coll, balanced: bool, trim: bool):
    """Pinned host micro-batches of this rank for optimizer step `step`, their real-token counts and
    the real-token count of every rank. The step's global batch (MICRO_PER_STEP x SEQS_PER_MICRO
    sequences) is the same whatever the number of ranks; with `balanced` it is dealt to the
    (rank, micro-step) bins by cost (nanoplm_b200.data.packing.balance_bins), otherwise in order."""
    import numpy as np
    import torch
    from nanoplm_b200.data.packing import balance_bins
    seqs = make_sequences(MICRO_PER_STEP * SEQS_PER_MICRO, 1234 + step)
    lens = np.fromiter((len(x) for x in seqs), np.int32, len(seqs))
    if balanced:
        bin_of, _ = balance_bins(lens, MICRO_PER_STEP, SEQS_PER_MICRO)
    else:
        bin_of = np.arange(len(seqs), dtype=np.int32) // SEQS_PER_MICRO
    per_rank_tokens = [int(sum(lens[bin_of == a * world + r].sum() for a in range(accum))) for r in range(world)]
    host, real = [], []
    for a in range(accum):
        idx = np.nonzero(bin_of == a * world + rank)[0]
        b = coll([{"input_ids": torch.from_numpy(seqs[i])} for i in idx])
        real.append(int(b["num_real_tokens"]))
        if not trim:                 # process the padding tail too (the reference's static shape)
            b.pop("num_real_tokens")
        b.pop("labels")              # masked_idx / masked_labels carry the same information
        host.append({k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in b.items()})
    return host, real, per_rank_tokens


def _pipeline_e2e(args, device, rank, world, accum, K, W):
    """The same metric through the user-facing pipeline: `run_pretraining` on a shard dataset
    (DataLoader workers, packing collator, pinned host -> device copy of every micro-batch, loss
    read back at every step). Returns (tokens/s over all ranks, ms per step, h2d bytes per step,
    d2h bytes per step) or None when --no-pipeline-e2e was given."""
    import torch
    import torch.distributed as dist
    from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig, PureTorchConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.runtime.pretrain import run_pretraining
    work = Path(tempfile.mkdtemp(prefix=f"nplm_own_r{rank}_"))
    n_train = (W + K + 1) * MICRO_PER_STEP * SEQS_PER_MICRO      # one spare step: the loader prefetches ahead
    if rank == 0 or world == 1:
        write_shard_dataset(work / "data", n_train, SEQS_PER_MICRO * world, seed=4321)
    if world > 1:
        paths = [str(work)]
        dist.broadcast_object_list(paths, src=0)
        work = Path(paths[0])
    cfg = PretrainingConfig(
        dataset_dir=str(work / "data"), ckp_dir=str(work / f"ckpt{rank}"), micro_batch_size=SEQS_PER_MICRO,
        num_epochs=1, warmup_ratio=0.05, optimizer="adamw", adam_learning_rate=1e-3,
        global_batch_size=MICRO_PER_STEP * SEQS_PER_MICRO * MAX_SEQ_LEN, bf16=True, tf32=True,
        mlm_probability=MLM_PROB, logging_steps=1, eval_steps=10 ** 9, save_steps=10 ** 9, seed=42,
        num_workers="auto", prefetch_factor=2, multi_gpu=world > 1, world_size=world, project_name="bench",
        fused_comm=not args.no_fused_comm, balance_ranks=not args.no_balance, metrics_jsonl=False,
        shard_params=bool(args.shard_params))
    pt = PureTorchConfig(use_compile=False, use_packing=True, target_packed_rows=TARGET_ROWS)
    torch.manual_seed(42)
    model = ProtEncoderMLM(ModelConfig(**MODEL), ProtTokenizer())
    st = {"t0": None, "e0": None, "ms": None, "tok": 0.0, "h2d": 0, "d2h": 0}

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def on_step(info: dict) -> None:
        n = info["global_step"]
        if n == W:
            sync_all()
            st["e0"] = torch.cuda.Event(enable_timing=True)
            st["e0"].record()
            st["t0"] = time.perf_counter()
        elif W < n <= W + K:
            st["tok"] += info["tokens"]
            st["h2d"] += info["h2d_bytes"]
            st["d2h"] += info["d2h_bytes"]
            if n == W + K:
                e1 = torch.cuda.Event(enable_timing=True)
                e1.record()
                sync_all()
                st["ms"] = max(st["e0"].elapsed_time(e1), 1e3 * (time.perf_counter() - st["t0"]))

    run_pretraining(model, cfg, pt, None, max_steps=W + K, on_step=on_step, final_checkpoint=False)
    t = torch.tensor([st["ms"] or 0.0, st["tok"]], dtype=torch.float64, device=device)
    if world > 1:
        mx = t[:1].clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(t[1:])
        t[0] = mx[0]
    ms, tokens = float(t[0]), float(t[1])
    if ms <= 0:
        return None
    return tokens / (ms / 1e3), ms / K, st["h2d"] // K, st["d2h"] // K


def run_own(args) -> dict:
    import statistics
    import torch
    import torch.distributed as dist
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime.pretrain import TrainStep, init_distributed, move_batch, set_seed
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    device, rank, world, local_rank = init_distributed(True)
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}; launch with torch.distributed.run")
    if MICRO_PER_STEP % world:
        raise SystemExit("gpus must divide 16")
    accum = MICRO_PER_STEP // world
    K, W = args.steps, args.warmup
    K_nt = 0 if (args.no_trim or args.variant != "default") else min(K, 2)   # extra steps over the full static shape
    set_seed(42)
    tok = ProtTokenizer()
    model_kw = dict(MODEL)
    if args.variant == "moe":        # every 2nd MLP -> 64 SwiGLU experts (I = 512), top-2
        from nanoplm_b200.config.schema import MoEConfig
        model_kw["moe"] = MoEConfig(num_experts=64, top_k=2, expert_intermediate_size=512, every_n_layers=2)
    elif args.variant == "conv_mhc":  # varlen depthwise conv (k = 7) + 4 hyper-connection streams
        model_kw.update(conv_kernel_size=7, mhc_streams=4)
    elif args.variant == "fp8":
        from nanoplm_b200.ops import functional as _ops
        _ops.set_fp8(True)
    model = ProtEncoderMLM(ModelConfig(**model_kw), tok)
    engine_cls = ShardedEngine
    if args.shard_params and world > 1:
        from nanoplm_b200.parallel.param_sharded import ParamShardedEngine
        engine_cls = ParamShardedEngine
    if args.variant == "moe" and world > 1:
        # expert parallelism: every rank keeps 64 / world experts, rows travel over peer memory
        from nanoplm_b200.parallel.expert_engine import ExpertParallelEngine, shard_model_experts
        shard_model_experts(model, dist.group.WORLD)
        engine_cls = ExpertParallelEngine
    engine = engine_cls(model, AdamWHyper(lr=1e-3, max_grad_norm=1.0), device,
                        compute_dtype=torch.bfloat16, fused_comm=not args.no_fused_comm)
    model.train()
    total_steps = W + 2 * K + K_nt
    sched = WarmupLinearSchedule(1e-3, max(1, total_steps // 20), total_steps * 50)
    stepper = TrainStep(model, engine, sched, device)
    balanced = world > 1 and not args.no_balance

    coll = PackingCollator(tok, MAX_SEQ_LEN, MLM_PROB, target_rows=TARGET_ROWS, batch_size=SEQS_PER_MICRO,
                           seed=99 + rank)
    steps_host, steps_tok, rank_tok = [], [], []
    for s in range(W + K):
        host, real, per_rank = _step_batches(s, rank, world, accum, coll, balanced, trim=not args.no_trim)
        steps_host.append(host)
        steps_tok.append(sum(real))
        rank_tok.append(per_rank)
    nt_host = [_step_batches(W + K + s, rank, world, accum, coll, balanced, trim=False) for s in range(K_nt)]

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the timed steps' batches go to the device BEFORE the warm-up steps: allocating them afterwards took
    # cached blocks away from the first timed step, which then paid for new device allocations
    timed_host = steps_host[W:]
    timed_dev = [[move_batch(b, device) for b in st] for st in timed_host]
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()              # the process starts during the warm-up, its samples count from begin()
    for s in range(W):
        stepper.step_from_host(steps_host[s])
    tokens_timed = sum(steps_tok[W:])
    tok_t = torch.tensor([float(tokens_timed)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(tok_t)
    global_tokens = float(tok_t.item())

    # ---- device-timed region ------------------------------------------------------------
    if engine.fused is not None:
        engine.fused.timing, engine.fused.tail_events = True, []
    sync_all()
    if sampler:
        sampler.begin()
    launches0 = _lib.launches()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
    marks[0].record()
    for i, st in enumerate(timed_dev):
        stepper.step_on_device(st)
        marks[i + 1].record()
    sync_all()
    ms = marks[0].elapsed_time(marks[-1])
    step_ms = [marks[i].elapsed_time(marks[i + 1]) for i in range(K)]
    launches = _lib.launches() - launches0
    clocks = sampler.stop() if sampler else None
    tail_ms = 0.0
    if engine.fused is not None:
        engine.fused.timing = False
        tails = [a.elapsed_time(b) for a, b in engine.fused.tail_events]
        tail_ms = sum(tails) / max(1, len(tails))

    # ---- the optimizer step's own arithmetic (AdamW on this rank's slice, no communication) ------
    from nanoplm_b200.ops import kernels as Kn
    g = torch.zeros(engine.shard, dtype=torch.float32, device=device)
    o = torch.empty(engine.shard, dtype=torch.bfloat16, device=device)
    ssq = torch.ones(1, dtype=torch.float32, device=device)
    pm, pv, pp_ = (torch.zeros_like(g) for _ in range(3))
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(4):
        if it == 1:
            a0.record()
        Kn.adamw_(pp_, pm, pv, g, o, engine._hyper_dev[0], ssq, zero_grad=False)
    a1.record()
    torch.cuda.synchronize()
    local_opt_ms = a0.elapsed_time(a1) / 3
    del g, o, pm, pv, pp_

    # ---- TrainStep from pinned host memory (H2D every micro-batch, loss read back every step) ---
    stepper.h2d_bytes = stepper.d2h_bytes = 0
    sync_all()
    t0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    last_loss = None
    for st in timed_host:
        last_loss = stepper.step_from_host(st)
    g1.record()
    sync_all()
    ts_ms = max(g0.elapsed_time(g1), 1e3 * (time.perf_counter() - t0))
    ts_h2d, ts_d2h = stepper.h2d_bytes // K, stepper.d2h_bytes // K

    # ---- the same steps over the full static shape (padding tail not cut off) -------------------
    nt_ms, nt_tokens = 0.0, 0.0
    if K_nt:
        nt_dev = [[move_batch(b, device) for b in h] for h, _, _ in nt_host]
        nt_tokens = float(sum(sum(r) for _, r, _ in nt_host))
        stepper.step_on_device(nt_dev[0])          # shapes change: one untimed step first
        sync_all()
        n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0.record()
        for st in nt_dev:
            stepper.step_on_device(st)
        n1.record()
        sync_all()
        nt_ms = n0.elapsed_time(n1)

    t = torch.tensor([ms, ts_ms, nt_ms, tail_ms, max(step_ms), -min(step_ms), -tail_ms], dtype=torch.float64,
                     device=device)
    nt_tok_t = torch.tensor([nt_tokens], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nt_tok_t)
    ms, ts_ms, nt_ms, tail_max_ms, tail_ms = float(t[0]), float(t[1]), float(t[2]), float(t[3]), -float(t[6])
    _lib.check_status()
    fused_on = engine.fused is not None
    n_params = engine.num_parameters()
    loaded = [Path(p).name for p in _lib.loaded_libraries()]
    overlapped = engine.fused.overlapped_bytes if fused_on else 0
    sharded_params = type(engine).__name__ == "ParamShardedEngine"
    gathered_bytes = engine.gathered_parameter_bytes() if sharded_params else 0

    # ---- end to end through the pipeline ------------------------------------------------------------
    moe_dropped = sum(m.dropped_rows() for m in model.modules() if hasattr(m, "dropped_rows"))
    del stepper, engine, model, timed_dev
    torch.cuda.empty_cache()
    pipe = None
    if not args.no_pipeline_e2e and args.variant == "default" and not args.no_trim:
        pipe = _pipeline_e2e(args, device, rank, world, accum, K, W)

    value = global_tokens / (ms / 1e3)
    e2e = {"value": global_tokens / (ts_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": ts_h2d,
           "d2h_bytes_per_step": ts_d2h, "ms_per_step": ts_ms / K,
           "path": "TrainStep.step_from_host on micro-batches collated ahead of time (pinned host memory)"}
    if pipe is not None:
        e2e = {"value": pipe[0], "unit": "tokens/s", "h2d_bytes_per_step": pipe[2], "d2h_bytes_per_step": pipe[3],
               "ms_per_step": pipe[1],
               "path": "run_pretraining on a shard dataset: DataLoader workers + packing collator + balanced "
                       "batch sampler, pinned host -> device copy of every micro-batch, loss and gradient norm "
                       "read back at every step",
               "trainstep_from_host": {"value": global_tokens / (ts_ms / 1e3), "ms_per_step": ts_ms / K,
                                       "h2d_bytes_per_step": ts_h2d, "d2h_bytes_per_step": ts_d2h}}
    spread = [max(r) / (sum(r) / len(r)) for r in rank_tok[W:]]
    res = {"metric": "mlm_pretrain_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
           "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None, "dtype": "bf16",
           "data": "synthetic (seeded amino-acid sequences, random-init weights)", "impl": "own",
           "config": config_block(world, accum), "clocks": clocks, "e2e": e2e,
           "gpu_launches": launches, "final_loss": last_loss,
           "step_ms": {"min": -float(t[5]), "median": statistics.median(step_ms), "max": float(t[4]),
                       "rank0_all": [round(x, 2) for x in step_ms],
                       "note": "device time of every timed optimizer step; min / max over ranks, median of rank 0"},
           "exposed_comm_ms": max(0.0, tail_ms - local_opt_ms) if fused_on else (0.0 if world == 1 else None),
           "exposed_comm": {"optimizer_step_after_backward_ms": tail_ms,
                            "optimizer_step_after_backward_ms_slowest_wait": tail_max_ms,
                            "local_adamw_ms": local_opt_ms,
                            "overlapped_with_backward_bytes_per_rank": overlapped,
                            "definition": "CUDA-event time from the end of the last backward pass to the end of "
                                          "the optimizer step (barriers, remaining reduce-scatter, norm exchange, "
                                          "AdamW + parameter push), mean over the timed steps, on the rank where "
                                          "it is SHORTEST: the rank that reaches the step last waits for nobody, so "
                                          "its tail is the communication on the critical path; minus the time of "
                                          "the same AdamW arithmetic on this rank's slice alone. The longest tail "
                                          "over the ranks additionally contains the wait for the slowest rank."},
           "rank_real_tokens_max_over_mean": {"mean": sum(spread) / len(spread), "max": max(spread),
                                              "balanced_assignment": balanced},
           "raw_tokens_per_sec": K * MICRO_PER_STEP * TARGET_ROWS * MAX_SEQ_LEN / (ms / 1e3),
           "fused_comm": fused_on, "loaded_libs": loaded}
    if args.shard_params:
        res["shard_params"] = {"active": sharded_params,
                               "bf16_bytes_gathered_inside_gemms_per_rank_per_step": gathered_bytes,
                               "note": "parameters, their gradient reduction and optimizer state are split by row "
                                       "blocks over the ranks; the all-gather runs inside the first forward GEMM "
                                       "that uses a matrix (RoPE / SwiGLU / residual epilogues)"}
        res["config"]["parallelism"] = f"dp{world}-sharded-parameters"
    if K_nt and nt_ms > 0:
        res["no_trim_value"] = float(nt_tok_t.item()) / (nt_ms / 1e3)
        res["no_trim_ms_per_step"] = nt_ms / K_nt
        res["no_trim_note"] = (f"{K_nt} further steps with the padding tail left in place (the static shape the "
                               "reference computes over): like-for-like kernel speed, real tokens counted")
    if args.no_trim:
        res["config"]["padding_tail"] = "own arm run with --no-trim: its kernels cover the padding tail as well"
    if args.variant != "default":
        res["variant"] = args.variant
        res["config"]["model"] += {"moe": " + MoE (64 experts, top-2, I 512) on every 2nd layer",
                                   "conv_mhc": " + varlen depthwise conv (k 7) + 4 mHC streams",
                                   "fp8": " with e4m3 block128 linear layers (not the headline precision)"}[args.variant]
        res["parameters"] = n_params
        if args.variant == "moe":
            res["moe"] = {"expert_rows_dropped_on_rank0": int(moe_dropped),
                          "dispatch": ("per-tile arrival counters gate the grouped up-projection"
                                       if os.environ.get("NPLM_MOE_GATED", "1") != "0" else
                                       "flag barrier between dispatch and up-projection") if world > 1 else "local"}
            if world > 1:
                res["config"]["parallelism"] = (f"ep{world} (64 experts over {world} ranks, rows over peer memory) "
                                                f"x dp{world}-sharded-optimizer for the dense part")
        if args.variant == "fp8":
            res["dtype"] = "fp8-e4m3 linears, bf16 elsewhere"
    if world > 1:
        dist.destroy_process_group()
    return res if rank == 0 else {}


# ----------------------------------------------------------------------------------- reference arm
def _stub_missing_modules():
    """Placeholders for third-party packages the reference imports at module level but does not use
    on the pretraining path (they are absent from this image)."""
    import importlib
    import types
    for name, attrs in (("IPython", {"get_ipython": lambda: None}), ("h5py", {"File": object}),
                        ("Bio", {}), ("Bio.SeqIO", {})):
        try:
            importlib.import_module(name)
        except Exception:
            m = types.ModuleType(name)
            for k, v in attrs.items():
                setattr(m, k, v)
            sys.modules[name] = m
    if "Bio" in sys.modules and "Bio.SeqIO" in sys.modules:
        setattr(sys.modules["Bio"], "SeqIO", sys.modules["Bio.SeqIO"])


def run_reference(args) -> dict:
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "nanoplm").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref/nanoplm not installed on this machine"}
    import torch
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    os.environ["WANDB_MODE"] = "disabled"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        return {"impl": "reference", "unavailable": f"--gpus {args.gpus} but WORLD_SIZE is {world}"}
    accum = MICRO_PER_STEP // world
    K, W = args.steps, args.warmup
    work = Path(tempfile.mkdtemp(prefix=f"nplm_ref_r{rank}_"))
    os.chdir(work)                      # the reference opens output/logs/pipeline.log in the cwd on import
    sys.path.insert(0, str(ref_dir))
    _stub_missing_modules()
    try:
        import torch.distributed as dist
        import nanoplm.pretraining.pure_pipeline as pp
        from nanoplm.pretraining.config import PretrainingConfig, PureTorchConfig
        from nanoplm.pretraining.models.modern_bert.model import ProtModernBertMLMConfig
        from nanoplm.pretraining.models.modern_bert.pure_model import PureProtModernBertMLM
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference import failed: {type(exc).__name__}: {exc}"[:300]}

    n_train = (W + K) * accum * SEQS_PER_MICRO * world
    total_real = write_shard_dataset(work / "data", n_train, SEQS_PER_MICRO * world, seed=1234)
    cfg = PretrainingConfig(
        dataset_dir=str(work / "data"), ckp_dir=str(work / "ckpt"), micro_batch_size=SEQS_PER_MICRO,
        num_epochs=1, warmup_ratio=0.05, optimizer="adamw", adam_learning_rate=1e-3,
        global_batch_size=MICRO_PER_STEP * SEQS_PER_MICRO * MAX_SEQ_LEN, bf16=True, tf32=True,
        mlm_probability=MLM_PROB, logging_steps=1, eval_steps=10 ** 9, save_steps=10 ** 9, seed=42,
        num_workers="auto", prefetch_factor=2, multi_gpu=world > 1, world_size=world,
        project_name="bench")
    pt = PureTorchConfig(use_compile=True, use_packing=True, target_packed_rows=TARGET_ROWS)
    torch.manual_seed(42)
    model = PureProtModernBertMLM(ProtModernBertMLMConfig(
        hidden_size=MODEL["hidden_size"], intermediate_size=MODEL["intermediate_size"],
        num_hidden_layers=MODEL["num_hidden_layers"], num_attention_heads=MODEL["num_attention_heads"],
        vocab_size=32, max_position_embeddings=MODEL["max_position_embeddings"]))

    state = {"n": 0, "ms": None, "clocks": None}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    orig_step = torch.optim.AdamW.step

    def sync_all():
        if world > 1 and dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def timed_step(self, *a, **kw):
        out = orig_step(self, *a, **kw)
        state["n"] += 1
        if state["n"] == 1 and sampler:
            sampler.start()      # during the warm-up, as in the own arm: NVML start-up stays out of the timed steps
        if state["n"] == W:
            sync_all()
            if sampler:
                sampler.begin()
            ev0.record()
        elif state["n"] == W + K:
            ev1.record()
            sync_all()
            state["ms"] = ev0.elapsed_time(ev1)
            if sampler:
                state["clocks"] = sampler.stop()
        return out

    torch.optim.AdamW.step = timed_step
    # the final evaluation / checkpoint of the reference run after the timed steps are not needed
    try:
        pp.run_pure_pretraining(model, cfg, pt, None)
    except Exception as exc:  # noqa: BLE001
        if state["ms"] is None:
            return {"impl": "reference", "unavailable": f"reference run failed: {type(exc).__name__}: {exc}"[:300]}
    finally:
        torch.optim.AdamW.step = orig_step
    if state["ms"] is None:
        return {"impl": "reference", "unavailable": f"reference finished after {state['n']} optimizer steps, "
                                                    f"expected {W + K}"}
    ms = state["ms"]
    if world > 1 and dist.is_initialized():
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    tokens = total_real * K / (W + K)      # one epoch consumes every sequence once; K of W+K steps are timed
    value = tokens / (ms / 1e3)
    res = {"metric": "mlm_pretrain_tokens_per_sec", "value": value, "unit": "tokens/s", "n_gpus": world,
           "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16", "impl": "reference",
           "data": "synthetic (seeded amino-acid sequences, random-init weights)",
           "config": config_block(world, accum), "clocks": state["clocks"],
           "e2e": {"value": value, "unit": "tokens/s", "note": "the reference path already includes its "
                   "DataLoader, host->device copies and per-micro-step loss.item() reads"},
           "raw_tokens_per_sec": K * MICRO_PER_STEP * TARGET_ROWS * MAX_SEQ_LEN / (ms / 1e3)}
    return res if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("own", "reference"), default="own")
    ap.add_argument("--no-fused-comm", action="store_true", help="use NCCL collectives in the optimizer step")
    ap.add_argument("--no-trim", action="store_true",
                    help="own arm: also run the kernels over the padding tail of every flat micro-batch")
    ap.add_argument("--shard-params", action="store_true",
                    help="own arm, several GPUs: row-sharded parameters with the all-gather inside the GEMMs")
    ap.add_argument("--no-balance", action="store_true",
                    help="own arm, several GPUs: deal the step's sequences to ranks in order instead of by cost")
    ap.add_argument("--no-pipeline-e2e", action="store_true",
                    help="own arm: skip the run_pretraining end-to-end region (e2e then reports TrainStep from host)")
    ap.add_argument("--variant", choices=("default", "moe", "conv_mhc", "fp8"), default="default",
                    help="own arm only: optional model extensions (the headline number is 'default')")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    res = run_reference(args) if args.impl == "reference" else run_own(args)
    if res:
        sys.stdout.flush()
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
