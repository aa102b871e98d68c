"""Device time of one optimizer step of the default encoder (169 M parameters) with random
gradients already in place: sharded AdamW (fused P2P or NCCL step) and Muon / NorMuon (stacked
Newton-Schulz on the row-grouped GEMM, matrices split over the ranks).

    python -m nanoplm_b200.bench.optimizer_bench [--optimizer adamw|muon|normuon] [--steps 10]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 -m nanoplm_b200.bench.optimizer_bench --optimizer muon

CUDA events after warm-up, maximum over ranks; rank 0 prints one JSON object per optimizer.
The reference's Muon path needs the `dion` package (src/nanoplm/pretraining/optim.py:121-184).
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizer", default="adamw,muon,normuon")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--no-fused-comm", action="store_true",
                    help="library collectives instead of the peer-memory kernels (multi-GPU A/B)")
    ap.add_argument("--per-matrix", action="store_true",
                    help="Muon: orthogonalise matrix by matrix on every rank (no stacking, no split over ranks)")
    args = ap.parse_args()

    from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.parallel.muon import MuonEngine
    from nanoplm_b200.runtime.pretrain import init_distributed

    device, rank, world, _ = init_distributed(True)
    for name in args.optimizer.split(","):
        torch.manual_seed(0)
        model = ProtEncoderMLM(ModelConfig(hidden_size=1024, intermediate_size=2048, num_hidden_layers=args.layers,
                                           num_attention_heads=16, vocab_size=32, max_position_embeddings=1024), ProtTokenizer())
        hyper = AdamWHyper(lr=1e-3, max_grad_norm=1.0)
        if name == "adamw":
            eng = ShardedEngine(model, hyper, device, compute_dtype=torch.bfloat16,
                                fused_comm=world > 1 and not args.no_fused_comm)
        else:
            eng = MuonEngine(model, hyper, PretrainingConfig(dataset_dir="x", optimizer=name), device,
                             fused_comm=world > 1 and not args.no_fused_comm)
            if args.per_matrix:
                from nanoplm_b200.parallel.muon import _Stack
                eng.stacks = [_Stack([s], 0, 1) for s in eng.muon_slots]
        g = torch.Generator(device=device).manual_seed(1 + rank)

        def one():
            eng.main_grad.normal_(0.0, 1e-3, generator=g)
            return eng.step(1e-3, 1)

        for _ in range(args.warmup):
            one()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0 = _lib.launches()
        e0.record()
        for _ in range(args.steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        _lib.check_status()
        if rank == 0:
            print(json.dumps({"bench": "optimizer_step", "optimizer": name + (" (matrix by matrix, replicated)" if args.per_matrix and name != "adamw" else ""),
                              "n_gpus": world, "peer_memory_comm": getattr(eng, "fused", None) is not None,
                              "parameters": eng.num_parameters(), "ms_per_step": round(float(t), 3),
                              "own_kernel_launches_per_step": (_lib.launches() - n0) // args.steps,
                              "note": "includes filling the gradient buffer with random numbers"}), flush=True)
        del eng, model
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
