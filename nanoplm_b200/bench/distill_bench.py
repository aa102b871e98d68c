"""Throughput of one on-the-fly distillation step: frozen T5-style teacher forward (ProtT5-XL
encoder shape by default, random weights) + ProtX student forward / backward + AdamW.

    python -m nanoplm_b200.bench.distill_bench [--batch 64] [--max-len 512] [--steps 5] [--layers 24]
                                               [--sdpa-teacher]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 -m nanoplm_b200.bench.distill_bench       # N ranks, --batch sequences each

Device time by CUDA events after warm-up (maximum over the ranks); rank 0 prints one JSON object
with the tokens of all ranks. `--sdpa-teacher` runs the
teacher's attention through PyTorch SDPA with a dense bias instead of this package's kernel.
The reference runs the same loop with HF T5EncoderModel under fp16 autocast
(src/nanoplm/distillation/collator.py:60-81) and an HF Trainer around the student.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=24, help="teacher layers (24 = ProtT5-XL encoder)")
    ap.add_argument("--sdpa-teacher", action="store_true")
    ap.add_argument("--student", choices=("default", "conv_mhc"), default="conv_mhc")
    args = ap.parse_args()

    from nanoplm_b200.config.schema import StudentConfig, TeacherConfig
    from nanoplm_b200.data.synthetic import synthetic_sequences
    from nanoplm_b200.models.student import ProtX
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime.distill import DistillDataCollator, distillation_loss

    import os
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    torch.manual_seed(0)
    teacher = T5EncoderTeacher(TeacherConfig(num_layers=args.layers), seed=1).to(dev).to(torch.bfloat16)
    teacher.native_attention = not args.sdpa_teacher
    kw = dict(conv_kernel_size=7, mhc_streams=4) if args.student == "conv_mhc" else {}
    student = ProtX(StudentConfig(**kw))
    engine = ShardedEngine(student, AdamWHyper(lr=1e-3), dev, fused_comm=world > 1)
    coll = DistillDataCollator(True, args.max_len)
    seqs = synthetic_sequences(args.batch, 20, args.max_len - 1, seed=4 + rank)
    batch = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in coll([{"raw_sequence": s} for s in seqs]).items()}
    tokens = int(batch["attention_mask"].sum().item())

    def step():
        engine.begin_last_microstep()       # one micro-batch per step: the reduction overlaps its backward pass
        loss = distillation_loss(student, batch, teacher)
        loss.backward()
        engine.step(1e-3, 1)
        return loss

    def teacher_only():
        with torch.no_grad():
            teacher(batch["teacher_input_ids"], batch["teacher_attention_mask"], lengths=batch.get("teacher_lengths"))

    def timed(fn, n):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / n], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_step = timed(step, args.steps)
    ms_teacher = timed(teacher_only, args.steps)
    _lib.check_status()
    tt = torch.tensor([float(tokens)], device=dev)
    if world > 1:
        dist.all_reduce(tt)
    tokens = int(tt.item())
    if rank == 0:
        print(json.dumps({"bench": "distillation_step", "n_gpus": world, "teacher_layers": args.layers,
                          "teacher_attention": "sdpa" if args.sdpa_teacher else "tcgen05 bias kernel",
                          "student": args.student, "batch_per_rank": args.batch, "max_len": args.max_len,
                          "real_tokens": tokens, "ms_per_step": round(ms_step, 2),
                          "ms_teacher_forward": round(ms_teacher, 2), "fused_comm": engine.fused is not None,
                          "real_tokens_per_sec": round(tokens / ms_step * 1e3, 0)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
