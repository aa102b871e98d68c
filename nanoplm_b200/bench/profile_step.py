"""One profiled training micro-step of the flagship encoder, bracketed by cudaProfilerStart/Stop.

    python -m nanoplm_b200.bench.profile_step [--tokens-rows 128] [--layers 16] [--optimizer-step]

Meant to run under `ncu --profile-from-start off ...` (launch list with gpu__time_duration.sum, or
a full-section capture of one kernel with -k on a reduced --tokens-rows / --layers). Without ncu it
prints the CUDA-event time of the profiled region.
"""
from __future__ import annotations

import argparse

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-rows", type=int, default=128, help="packed rows of 512 tokens")
    ap.add_argument("--seqs", type=int, default=208)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--optimizer-step", action="store_true")
    ap.add_argument("--variant", choices=("default", "moe", "conv_mhc"), default="default")
    ap.add_argument("--no-trim", action="store_true", help="run the kernels over the padding tail as well")
    ap.add_argument("--gaps", action="store_true",
                    help="trace the step with torch.profiler and report the GPU idle time between kernels")
    args = ap.parse_args()

    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime.pretrain import model_inputs, move_batch

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    tok = ProtTokenizer()
    extra = {}
    if args.variant == "moe":
        from nanoplm_b200.config.schema import MoEConfig
        extra["moe"] = MoEConfig(num_experts=64, top_k=2, expert_intermediate_size=512, every_n_layers=2)
    elif args.variant == "conv_mhc":
        extra.update(conv_kernel_size=7, mhc_streams=4)
    model = ProtEncoderMLM(ModelConfig(hidden_size=1024, intermediate_size=2048, num_hidden_layers=args.layers,
                                       num_attention_heads=16, max_position_embeddings=1024, **extra), tok)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.02)
            if hasattr(layer.mlp, "Wo"):
                layer.mlp.Wo.weight.normal_(0, 0.02)
            else:
                layer.mlp.experts_Wo.normal_(0, 0.02)
    engine = ShardedEngine(model, AdamWHyper(lr=1e-4), dev)
    model.train()
    seqs = synthetic_token_sequences(args.seqs, 19, 511, seed=7)
    coll = PackingCollator(tok, 512, 0.15, target_rows=args.tokens_rows, batch_size=args.seqs, seed=3)
    b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
    n_real = b.pop("num_real_tokens")
    b.pop("labels")
    batch = model_inputs(move_batch(b, dev))
    if not args.no_trim:
        batch["num_real_tokens"] = int(n_real)   # the padding tail is cut off before the first kernel

    def micro():
        out = model(**batch)
        out["loss"].backward()
        if args.optimizer_step:
            engine.step(1e-4, 1)

    for _ in range(args.warmup):
        micro()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof = None
    if args.gaps:
        from torch.profiler import ProfilerActivity, profile
        prof = profile(activities=[ProfilerActivity.CUDA])
        prof.__enter__()
    torch.cuda.profiler.start()
    e0.record()
    micro()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    if prof is not None:
        prof.__exit__(None, None, None)
        _report_gaps(prof)
    _lib.check_status()
    print(f"profiled micro-step: {e0.elapsed_time(e1):.3f} ms, {args.tokens_rows * 512} flat tokens, "
          f"{args.layers} layers, kernels launched by this package so far: {_lib.launches()}")


def _report_gaps(prof) -> None:
    """Union of the kernel intervals of the trace against its span: what is left is launch latency
    and dependencies between consecutive kernels."""
    ev = sorted((e.time_range.start, e.time_range.end) for e in prof.events()
                if e.device_type == torch.autograd.DeviceType.CUDA)
    if not ev:
        print("gaps: the trace holds no device events")
        return
    busy, gaps = 0.0, []
    cur_s, cur_e = ev[0]
    for s, e in ev[1:]:
        if s > cur_e:
            gaps.append(s - cur_e)
            busy += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    busy += cur_e - cur_s
    span = ev[-1][1] - ev[0][0]
    gaps.sort()
    med = gaps[len(gaps) // 2] if gaps else 0.0
    print(f"gaps: {len(ev)} device activities, span {span / 1e3:.2f} ms, busy {busy / 1e3:.2f} ms, "
          f"idle {(span - busy) / 1e3:.2f} ms in {len(gaps)} gaps (median {med:.1f} us, "
          f"max {gaps[-1] if gaps else 0.0:.1f} us)")


if __name__ == "__main__":
    main()
