"""Multi-GPU microbenchmarks of the fused compute + communication kernels next to the NCCL path
they replace. One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 -m nanoplm_b200.bench.comm_bench [--tokens 65536] [--what ag,agepi,opt,moe]

Every number is device time (CUDA events on the launching stream, barrier + synchronize on both
sides, warm-up first), the maximum over the ranks. Rank 0 prints one JSON object per measurement
with the roofline fraction  max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s) / time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

BF = torch.bfloat16
NVLINK_GBS = 770.0          # measured peer-copy bandwidth per direction per GPU on this pool


def _timed(fn, iters: int, warmup: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bench_ag_gemm(T, rank, world, dev, peaks):
    """QKV and MLP-up projections with the weight row-sharded over the ranks."""
    from nanoplm_b200.comm.fused_optimizer import SymmetricBuffer
    from nanoplm_b200.ops import kernels as K
    for name, N, Kd in [("qkv", 3072, 1024), ("mlp_up", 4096, 1024)]:
        rows = N // world
        if rows % 128:
            continue
        x = torch.randn(T, Kd, device=dev).to(BF)
        sb = SymmetricBuffer(N * Kd, BF, dev, dist.group.WORLD)
        full = sb.tensor.view(N, Kd)
        full.normal_(0, 0.05)
        flags = torch.zeros(8, dtype=torch.int32, device=dev)
        out = torch.empty(T, N, dtype=BF, device=dev)
        shard = full[rank * rows:(rank + 1) * rows].clone()
        gathered = torch.empty(N, Kd, dtype=BF, device=dev)
        torch.cuda.synchronize()
        dist.barrier()

        def fused():
            K.gemm_ag(x, full, sb.ptr_array, rank, world, flags, out=out)

        def nccl():
            dist.all_gather_into_tensor(gathered, shard)
            K.gemm(x, gathered, out=out)

        def plain():
            K.gemm(x, gathered, out=out)

        ms_f = _timed(fused, 20, 5, dev)
        ms_n = _timed(nccl, 20, 5, dev)
        ms_p = _timed(plain, 20, 5, dev)
        flops = 2.0 * T * N * Kd
        link_bytes = (world - 1) * rows * Kd * 2
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"kernel": "ag_gemm_bf16", "shape": name, "M": T, "N": N, "K": Kd, "n_gpus": world,
                              "ms_fused": round(ms_f, 4), "ms_nccl_allgather_plus_gemm": round(ms_n, 4),
                              "ms_gemm_only": round(ms_p, 4), "tflops_fused": round(flops / ms_f / 1e9, 1),
                              "nvlink_bytes": link_bytes, "roofline_ms": round(t_roof, 4),
                              "fraction_of_roofline": round(t_roof / ms_f, 3)}), flush=True)


def bench_ag_epilogues(T, rank, world, dev, peaks):
    """The all-gather GEMM with the epilogues of the training path (RoPE for QKV, SwiGLU for MLP-up,
    residual add for the two output projections) next to the plain GEMM with the same epilogue."""
    from nanoplm_b200.comm.fused_optimizer import SymmetricBuffer
    from nanoplm_b200.ops import kernels as K
    pos = (torch.arange(T, device=dev) % 512).to(torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device=dev).float() / 64))
    fr = torch.outer(torch.arange(1024, device=dev).float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    cases = [("qkv_rope", 3072, 1024, K.EPI_ROPE), ("mlp_up_swiglu", 4096, 1024, K.EPI_SWIGLU),
             ("attn_out_add", 1024, 1024, K.EPI_ADD), ("mlp_down_add", 1024, 2048, K.EPI_ADD)]
    for name, N, Kd, epi in cases:
        rows = N // world
        if rows % 128 or (epi == K.EPI_SWIGLU and world % 2):
            continue
        x = torch.randn(T, Kd, device=dev).to(BF)
        sb = SymmetricBuffer(N * Kd, BF, dev, dist.group.WORLD)
        full = sb.tensor.view(N, Kd)
        full.normal_(0, 0.05)
        flags = torch.zeros(8, dtype=torch.int32, device=dev)
        out_cols = N // 2 if epi == K.EPI_SWIGLU else N
        out = torch.empty(T, out_cols, dtype=BF, device=dev)
        aux = None
        if epi == K.EPI_ADD:
            aux = torch.randn(T, N, device=dev).to(BF)
        elif epi == K.EPI_SWIGLU:
            aux = torch.empty(T, N, dtype=BF, device=dev)
        rope = (pos, cos, sin, 2048) if epi == K.EPI_ROPE else None
        torch.cuda.synchronize()
        dist.barrier()
        ms_f = _timed(lambda: K.gemm_ag(x, full, sb.ptr_array, rank, world, flags, epi=epi, out=out, aux=aux,
                                        rope=rope), 20, 5, dev)
        ms_p = _timed(lambda: K.gemm(x, full, epi=epi, out=out, aux=aux, rope=rope), 20, 5, dev)
        flops = 2.0 * T * N * Kd
        link_bytes = (world - 1) * rows * Kd * 2
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"kernel": "ag_gemm_bf16", "shape": name, "M": T, "N": N, "K": Kd, "n_gpus": world,
                              "ms_fused": round(ms_f, 4), "ms_gemm_only": round(ms_p, 4),
                              "tflops_fused": round(flops / ms_f / 1e9, 1), "nvlink_bytes": link_bytes,
                              "roofline_ms": round(t_roof, 4), "fraction_of_roofline": round(t_roof / ms_f, 3)}),
                  flush=True)


def bench_optimizer_comm(T, rank, world, dev, peaks):
    """The optimizer step's kernels on the default encoder's 169 M parameters, one by one: the
    reduce-scatter + norm kernel (pulls 1 / N of the fp32 gradients from every peer) and the AdamW +
    push kernel (writes the bf16 slice to every peer), with the achieved NVLink rate and the fraction
    of the link roofline, next to the whole fused step and the NCCL step it replaces."""
    from ctypes import c_int, c_longlong
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops._lib import ptr, stream_ptr
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    res = {}
    for fused in (True, False):
        torch.manual_seed(0)
        model = ProtEncoderMLM(ModelConfig(hidden_size=1024, intermediate_size=2048, num_hidden_layers=16,
                                           num_attention_heads=16, vocab_size=32, max_position_embeddings=1024),
                               ProtTokenizer())
        eng = ShardedEngine(model, AdamWHyper(lr=1e-3, max_grad_norm=1.0), dev, compute_dtype=BF, fused_comm=fused)
        eng.main_grad.normal_(0.0, 1e-3)
        res["fused_step" if fused else "nccl_step"] = _timed(lambda: eng.step(1e-3, 1), 10, 3, dev)
        if fused and eng.fused is not None:
            f = eng.fused
            L = f._lib
            res["rs_sumsq"] = _timed(lambda: L.nplm_rs_sumsq(f.grads.ptr_array, c_int(world), c_longlong(eng.lo),
                                                             c_longlong(eng.shard), ptr(f.shard_grad), ptr(f.partial),
                                                             stream_ptr()), 10, 3, dev)
            eng._fill_hyper(1e-3, 1.0)
            res["adamw_push"] = _timed(lambda: L.nplm_adamw_push(
                ptr(eng.master), ptr(eng.exp_avg), ptr(eng.exp_avg_sq), ptr(f.shard_grad), f.params.ptr_array,
                c_int(world), c_longlong(eng.lo), c_longlong(eng.shard), c_longlong(eng.decay_end),
                ptr(eng._hyper_dev[0]), ptr(f.local_slots), ptr(f.norm), stream_ptr()), 10, 3, dev)
            res["barrier"] = _timed(f.barrier, 20, 3, dev)
            shard = eng.shard
        del eng, model
        torch.cuda.empty_cache()
    if rank == 0:
        out = {"bench": "optimizer_step_communication", "n_gpus": world, "ms": {k: round(v, 4) for k, v in res.items()}}
        if "rs_sumsq" in res:
            rs_bytes = 4 * shard * (world - 1)            # remote fp32 gradient slices pulled by one rank
            push_bytes = 2 * shard * (world - 1)          # bf16 slice written to every peer
            hbm = peaks.get("hbm_gbs", 6538.6)
            rs_roof = max(rs_bytes / (NVLINK_GBS * 1e9), 4 * shard * (world + 1) / (hbm * 1e9)) * 1e3
            push_roof = max(push_bytes / (NVLINK_GBS * 1e9), (28 + 2) * shard / (hbm * 1e9)) * 1e3
            out["rs_sumsq"] = {"nvlink_bytes_in": rs_bytes, "nvlink_gbs": round(rs_bytes / res["rs_sumsq"] / 1e6, 1),
                               "roofline_ms": round(rs_roof, 4), "fraction_of_roofline": round(rs_roof / res["rs_sumsq"], 3)}
            out["adamw_push"] = {"nvlink_bytes_out": push_bytes,
                                 "nvlink_gbs": round(push_bytes / res["adamw_push"] / 1e6, 1),
                                 "roofline_ms": round(push_roof, 4),
                                 "fraction_of_roofline": round(push_roof / res["adamw_push"], 3)}
            out["note"] = ("roofline = max(NVLink bytes / 770 GB/s measured peer copy, local HBM bytes / measured "
                           "copy bandwidth); in training the reduce-scatter runs per parameter under the backward pass")
        print(json.dumps(out), flush=True)


def bench_moe_ep(T, rank, world, dev, peaks):
    """One MoE layer (64 experts, top-2, I = 512) forward + backward with the experts split over the
    ranks: peer-memory push / pull against the all-to-all restatement of the same layer."""
    from nanoplm_b200.config.schema import ModelConfig, MoEConfig
    from nanoplm_b200.models.moe import MoEMLP
    cfg = ModelConfig(hidden_size=1024, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=16,
                      moe=MoEConfig(num_experts=64, top_k=2, expert_intermediate_size=512, every_n_layers=2))
    torch.manual_seed(5)
    x = torch.randn(T, 1024, device=dev).to(BF).requires_grad_(True)
    gy = torch.randn(T, 1024, device=dev).to(BF)
    res = {}
    for name, device_path in [("peer_memory", True), ("all_to_all", False)]:
        torch.manual_seed(1)
        layer = MoEMLP(cfg, ep_group=dist.group.WORLD, device_path=device_path).to(dev).to(BF)
        with torch.no_grad():
            layer.experts_Wo.normal_(0, 0.02)

        def step():
            y, aux = layer(x)
            (y.float() * gy.float()).sum().add(aux).backward()

        res[name] = _timed(step, 5, 2, dev)
    if rank == 0:
        flops = 3 * 2.0 * T * 2 * (1024 * 1024 + 1024 * 512)
        # every assignment's row crosses NVLink four times (dispatch, combine and their gradients)
        link_bytes = 4 * T * 2 * 1024 * 2 * (world - 1) / world
        t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        print(json.dumps({"kernel": "moe_layer_expert_parallel_fwd_bwd", "tokens_per_rank": T, "n_gpus": world,
                          "ms_peer_memory": round(res["peer_memory"], 3),
                          "ms_all_to_all_baseline": round(res["all_to_all"], 3),
                          "roofline_ms": round(t_roof, 3),
                          "fraction_of_roofline": round(t_roof / res["peer_memory"], 3)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--what", default="ag,moe")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.utils.peaks import measured_peaks
    peaks = measured_peaks()
    for what in args.what.split(","):
        {"ag": bench_ag_gemm, "agepi": bench_ag_epilogues, "opt": bench_optimizer_comm,
         "moe": bench_moe_ep}[what](args.tokens, rank, world, dev, peaks)
    from nanoplm_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
