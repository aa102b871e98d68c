"""Per-kernel microbenchmarks on one GPU: this package's sm_100a kernels next to the library
call they replace (cuBLAS via torch.matmul, flash-attn 2 varlen), timed with CUDA events after
warm-up, inputs larger than L2 or an L2 flush between iterations.

    python -m nanoplm_b200.bench.kernel_bench [--tokens 65536] [--what gemm,attn,elementwise]

Prints one JSON object per measurement.
"""
from __future__ import annotations

import argparse
import json

import torch

BF = torch.bfloat16


def _flush_buf():
    return torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")


_PROFILE = [False]     # --profile: one warm-up and one timed launch per kernel (a short run for a profiler)


def time_fn(fn, iters=10, warmup=3, flush=None):
    if _PROFILE[0]:
        iters, warmup = 1, 1
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(T, peaks, sweep_splits=False):
    from nanoplm_b200.ops import kernels as k
    flush = _flush_buf()
    shapes = [  # (name, M, N, K, a_mn, b_mn, epi)
        ("qkv_fwd", T, 3072, 1024, False, False, k.EPI_STORE),
        ("attn_out_fwd_add", T, 1024, 1024, False, False, k.EPI_ADD),
        ("mlp_up_fwd_swiglu", T, 4096, 1024, False, False, k.EPI_SWIGLU),
        ("mlp_up_fwd", T, 4096, 1024, False, False, k.EPI_STORE),
        ("mlp_down_fwd_add", T, 1024, 2048, False, False, k.EPI_ADD),
        ("qkv_dgrad", T, 1024, 3072, False, True, k.EPI_STORE),
        ("mlp_up_dgrad", T, 1024, 4096, False, True, k.EPI_STORE),
        ("mlp_down_dgrad", T, 2048, 1024, False, True, k.EPI_STORE),
        ("qkv_wgrad", 3072, 1024, T, True, True, k.EPI_ATOMIC_F32),
        ("attn_out_wgrad", 1024, 1024, T, True, True, k.EPI_ATOMIC_F32),
        ("mlp_up_wgrad", 4096, 1024, T, True, True, k.EPI_ATOMIC_F32),
        ("mlp_down_wgrad", 1024, 2048, T, True, True, k.EPI_ATOMIC_F32),
    ]
    for name, M, N, K, a_mn, b_mn, epi in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda").to(BF)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda").to(BF)
        aux = torch.randn(M, N, device="cuda").to(BF) if epi in (k.EPI_ADD, k.EPI_SWIGLU) else None
        out = None
        splits = 1
        if epi == k.EPI_ATOMIC_F32:
            out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
            splits = k.wgrad_splits(M, N, K)
        for bn in (256, 128):
            if epi == k.EPI_ATOMIC_F32:
                splits = k.wgrad_splits(M, N, K, bn)
            ms = time_fn(lambda: k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=epi, out=out, aux=aux,
                                        splits=splits, bn=bn), flush=flush)
            tf = 2.0 * M * N * K / ms / 1e9
            print(json.dumps({"kernel": "gemm_bf16_tcgen05", "case": name, "bn": bn, "splits": splits,
                              "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
                              "frac_of_measured_bf16": round(tf / peaks["bf16_tflops"], 3)}))
        if not (a_mn and not b_mn):
            sp = k.wgrad_splits(M, N, K, 256) if epi == k.EPI_ATOMIC_F32 else 1
            ms = time_fn(lambda: k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=epi, out=out, aux=aux,
                                        splits=sp, bn=256, pair=True), flush=flush)
            tf = 2.0 * M * N * K / ms / 1e9
            print(json.dumps({"kernel": "gemm_bf16_tcgen05_cta_pair", "case": name, "bn": 256, "splits": sp,
                              "M": M, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
                              "frac_of_measured_bf16": round(tf / peaks["bf16_tflops"], 3)}))
        if epi == k.EPI_ATOMIC_F32 and sweep_splits:
            for pr in (False, True):
                for sp in (0, 1, 2, 3, 4, 6, 8, 12, 16):
                    ms = time_fn(lambda: k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, epi=epi, out=out, splits=sp, bn=256,
                                                pair=pr), flush=flush)
                    tf = 2.0 * M * N * K / ms / 1e9
                    print(json.dumps({"kernel": "gemm_bf16_tcgen05" + ("_cta_pair" if pr else ""), "case": name,
                                      "bn": 256, "splits": sp if sp else "stream-k", "M": M, "N": N, "K": K,
                                      "ms": round(ms, 4), "tflops": round(tf, 1),
                                      "frac_of_measured_bf16": round(tf / peaks["bf16_tflops"], 3)}))
        af = a.t() if a_mn else a
        bf_ = b if b_mn else b.t()
        ms = time_fn(lambda: torch.matmul(af, bf_), flush=flush)
        tf = 2.0 * M * N * K / ms / 1e9
        print(json.dumps({"kernel": "cublas(torch.matmul)", "case": name, "ms": round(ms, 4),
                          "tflops": round(tf, 1)}))
    k.check_status()


def _packed_batch(T, lo=20, hi=512, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens, tot = [], 0
    while tot < T:
        n = int(torch.randint(lo, hi + 1, (1,), generator=g))
        n = min(n, T - tot)
        lens.append(n)
        tot += n
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return lens, torch.tensor(cu, dtype=torch.int32, device="cuda")


def bench_attn(T, peaks):
    from nanoplm_b200.ops import kernels as k
    H, D = 16, 64
    lens, cu = _packed_batch(T)
    flops_pairs = {-1: sum(n * n for n in lens),
                   64: sum(sum(min(n, i + 65) - max(0, i - 64) for i in range(n)) for n in lens)}
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    ss, se = k.seq_bounds(cu, T)
    flush = _flush_buf()
    try:
        from flash_attn import flash_attn_varlen_func
    except Exception:  # pragma: no cover
        flash_attn_varlen_func = None
    for window in (-1, 64):
        fwd_flops = 4.0 * flops_pairs[window] * D * H
        for impl in ("ws", "single"):
            ms = time_fn(lambda: k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl=impl), flush=flush)
            print(json.dumps({"kernel": "fa_varlen_fwd", "impl": impl, "window": window, "T": T,
                              "ms": round(ms, 4), "tflops": round(fwd_flops / ms / 1e9, 1)}), flush=True)
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, 0.125)
        for impl in ("ws", "single"):
            ms = time_fn(lambda: k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl=impl), flush=flush)
            print(json.dumps({"kernel": "fa_varlen_bwd", "impl": impl, "window": window, "T": T,
                              "ms": round(ms, 4), "tflops": round(2.5 * fwd_flops / ms / 1e9, 1)}), flush=True)
        if flash_attn_varlen_func is not None:
            q, kk, v = qkv.view(T, 3, H, D).unbind(1)
            q = q.contiguous().requires_grad_(True)
            kk = kk.contiguous().requires_grad_(True)
            v = v.contiguous().requires_grad_(True)
            mx = max(lens)
            ws = (-1, -1) if window < 0 else (window, window)
            f = lambda: flash_attn_varlen_func(q, kk, v, cu, cu, mx, mx, softmax_scale=0.125, window_size=ws)
            ms = time_fn(f, flush=flush)
            print(json.dumps({"kernel": "flash_attn2_fwd", "window": window, "ms": round(ms, 4),
                              "tflops": round(fwd_flops / ms / 1e9, 1)}))
            o = f()
            do = dout.view(T, H, D)
            ms = time_fn(lambda: torch.autograd.grad(o, (q, kk, v), do, retain_graph=True), flush=flush)
            print(json.dumps({"kernel": "flash_attn2_bwd", "window": window, "ms": round(ms, 4),
                              "tflops": round(2.5 * fwd_flops / ms / 1e9, 1)}))
    k.check_status()


def bench_attn_ws(T, peaks):
    """Only the warp-specialised attention kernels (a small, library-free target for profilers)."""
    from nanoplm_b200.ops import kernels as k
    H, D = 16, 64
    lens, cu = _packed_batch(T)
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    ss, se = k.seq_bounds(cu, T)
    flush = _flush_buf()
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32).cuda()
    pos = torch.cat([pos, torch.zeros(T - pos.numel(), dtype=torch.int32, device="cuda")])[:T].contiguous()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(1024, device="cuda").float(), inv)
    rope = (pos, fr.cos().contiguous(), fr.sin().contiguous())
    for window in (-1, 64):
        ms = time_fn(lambda: k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws"), iters=5, flush=flush)
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        ms_b = time_fn(lambda: k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl="ws"), iters=5,
                       flush=flush)
        ms_d = time_fn(lambda: k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl="ws",
                                        deterministic=True), iters=5, flush=flush)
        # as in training: q / k were rotated by the QKV GEMM, dQ / dK are rotated back inside the backward
        # kernels, rowsum(dO * O) comes from the output projection's data-gradient GEMM
        delta = torch.zeros(H, T, device="cuda")
        ms_r = time_fn(lambda: k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl="ws",
                                        rope=rope, delta=delta, delta_ready=True), iters=5, flush=flush)
        print(json.dumps({"kernel": "fa_varlen_ws", "window": window, "T": T, "fwd_ms": round(ms, 4),
                          "bwd_ms": round(ms_b, 4), "bwd_deterministic_ms": round(ms_d, 4),
                          "bwd_fused_rope_delta_ready_ms": round(ms_r, 4)}), flush=True)
    k.check_status()


def bench_elementwise(T, peaks):
    from nanoplm_b200.ops import kernels as k
    C, I = 1024, 2048
    x = torch.randn(T, C, device="cuda").to(BF)
    w = torch.ones(C, device="cuda").to(BF)
    dy = torch.randn(T, C, device="cuda").to(BF)
    hbm = peaks["hbm_gbs"]

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "GBps": round(gbs, 1),
                          "frac_of_measured_hbm": round(gbs / hbm, 3)}))

    ms = time_fn(lambda: k.norm_fwd(x, w, 1e-5))
    report("layernorm_fwd", ms, 2 * T * C * 2)
    y, mean, rstd = k.norm_fwd(x, w, 1e-5)
    dw = torch.zeros(C, device="cuda")
    ms = time_fn(lambda: k.norm_bwd(dy, x, w, mean, rstd, dres=dy, dw=dw))
    report("layernorm_bwd", ms, 4 * T * C * 2)
    pre = torch.randn(T, 2 * I, device="cuda").to(BF)
    ms = time_fn(lambda: k.swiglu_fwd(pre))
    report("swiglu_fwd", ms, 3 * T * I * 2)
    do = torch.randn(T, I, device="cuda").to(BF)
    ms = time_fn(lambda: k.swiglu_bwd(pre, do))
    report("swiglu_bwd", ms, 5 * T * I * 2)
    qkv = torch.randn(T, 3 * C, device="cuda").to(BF)
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    cos = torch.randn(1024, 32, device="cuda")
    sin = torch.randn(1024, 32, device="cuda")
    ms = time_fn(lambda: k.rope_(qkv, pos, cos, sin, 16, 64))
    report("rope", ms, 4 * T * C * 2)
    n = 168_888_352
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, dtype=BF, device="cuda")
    hyper = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0, 1.0], device="cuda")
    ss = torch.ones(1, device="cuda")
    ms = time_fn(lambda: k.adamw_(p, m, v, g, pb, hyper, ss))
    report("adamw", ms, n * (4 * 4 + 3 * 4 + 2))
    k.check_status()


def bench_fp8(T, peaks):
    """e4m3 block-scaled GEMM (per-K-block promotion) next to the bf16 tcgen05 GEMM, and the
    quantisation kernels."""
    from nanoplm_b200.ops import fp8
    from nanoplm_b200.ops import kernels as k
    flush = _flush_buf()
    for name, N, K in [("qkv_fwd", 3072, 1024), ("mlp_up_fwd", 4096, 1024), ("mlp_down_fwd", 1024, 2048)]:
        x = torch.randn(T, K, device="cuda").to(BF)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(BF)
        qx, qw = fp8.quant_rows(x), fp8.quant_tile(w, transpose=False, block=True)
        out = torch.empty(T, N, dtype=BF, device="cuda")
        ms8 = time_fn(lambda: fp8.gemm_fp8(qx, qw, out=out), flush=flush)
        ms16 = time_fn(lambda: k.gemm(x, w, out=out), flush=flush)
        msq = time_fn(lambda: fp8.quant_rows(x), flush=flush)
        fl = 2.0 * T * N * K
        print(json.dumps({"kernel": "gemm_fp8_block128", "shape": name, "M": T, "N": N, "K": K,
                          "ms_fp8": round(ms8, 4), "tflops_fp8": round(fl / ms8 / 1e9, 1),
                          "ms_bf16": round(ms16, 4), "tflops_bf16": round(fl / ms16 / 1e9, 1),
                          "ms_quant_rows": round(msq, 4),
                          "quant_gbs": round(T * K * 3 / msq / 1e6, 1)}), flush=True)


def bench_moe(T, peaks):
    """Grouped tcgen05 GEMM over 64 experts (I = 512, top-2) next to a loop of per-expert GEMMs, and
    the whole device-side MoE layer forward + backward."""
    from nanoplm_b200.ops import kernels as k
    from nanoplm_b200.ops import moe as M
    flush = _flush_buf()
    E, top_k, C, I = 64, 2, 1024, 512
    torch.manual_seed(0)
    experts = torch.randint(0, E, (T, top_k), device="cuda", dtype=torch.int32)
    comm = M.MoEComm(C, E, top_k)
    plan = M.make_plan(comm, experts)
    xs = torch.randn(plan.cap, C, device="cuda").to(BF)
    Wi = (torch.randn(E, 2 * I, C, device="cuda") * 0.03).to(BF)
    Wo = (torch.randn(E, C, I, device="cuda") * 0.03).to(BF)
    pre = torch.empty(plan.cap, 2 * I, dtype=BF, device="cuda")
    ms_up = time_fn(lambda: M.gemm_grouped(xs, Wi, plan.tile_group, epi=k.EPI_SWIGLU, aux=pre), flush=flush)
    off = plan.group_off.cpu().tolist()
    rows = off[-1]

    def loop():
        for e in range(E):
            if off[e + 1] > off[e]:
                k.gemm(xs[off[e]:off[e + 1]], Wi[e], epi=k.EPI_SWIGLU, aux=pre[off[e]:off[e + 1]])

    ms_loop = time_fn(loop, flush=flush)
    fl = 2.0 * rows * 2 * I * C
    print(json.dumps({"kernel": "gemm_grouped_swiglu", "experts": E, "rows": rows, "N": 2 * I, "K": C,
                      "ms_grouped": round(ms_up, 4), "tflops_grouped": round(fl / ms_up / 1e9, 1),
                      "ms_per_expert_loop": round(ms_loop, 4)}), flush=True)
    x = torch.randn(T, C, device="cuda").to(BF).requires_grad_(True)
    logits = torch.randn(T, E, device="cuda").to(BF).requires_grad_(True)
    Wi.requires_grad_(True)
    Wo.requires_grad_(True)
    gy = torch.randn(T, C, device="cuda").to(BF)

    def layer():
        y, aux = M.moe_mlp(x, logits, Wi, Wo, top_k, comm)
        (y.float() * gy.float()).sum().add(aux).backward()

    ms_layer = time_fn(layer, iters=5, flush=flush)
    flops = 3 * 2.0 * T * top_k * (2 * I * C + C * I)
    print(json.dumps({"kernel": "moe_layer_fwd_bwd", "tokens": T, "experts": E, "top_k": top_k,
                      "ms": round(ms_layer, 3), "expert_tflops": round(flops / ms_layer / 1e9, 1)}), flush=True)


def bench_misc(T, peaks):
    """The small kernels around the encoder that the other cases do not launch: fused MLM-head
    cross-entropy (forward / backward), Philox masking, the teacher's bias attention, masked MSE, the
    optimizer-step communication kernels on one rank (their local memory traffic) and the Muon
    momentum / apply kernels."""
    import ctypes
    from ctypes import c_int, c_longlong
    from nanoplm_b200.ops import kernels as k
    from nanoplm_b200.ops._lib import lib, ptr, stream_ptr
    hbm = peaks["hbm_gbs"]
    flush = _flush_buf()

    def report(name, ms, nbytes, **extra):
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "GBps": round(gbs, 1),
                          "frac_of_measured_hbm": round(gbs / hbm, 3), **extra}), flush=True)

    C, V = 1024, 32
    n = T * 3 // 10                                        # masked positions of a 30 % MLM batch
    h = torch.randn(n, C, device="cuda").to(BF)
    W = (torch.randn(V, C, device="cuda") * 0.03).to(BF)
    bias = torch.zeros(V, device="cuda").to(BF)
    labels = torch.randint(0, V, (n,), device="cuda")
    inv = torch.full((1,), 1.0 / n, device="cuda")
    ms = time_fn(lambda: k.ce_fwd(h, W, bias, labels, inv), flush=flush)
    report("ce_fwd", ms, n * C * 2 + n * 32 * 4, rows=n)
    _, dlogits, _ = k.ce_fwd(h, W, bias, labels, inv)
    dW = torch.zeros(V, C, device="cuda")
    db = torch.zeros(V, device="cuda")
    gs = torch.ones(1, device="cuda")
    ms = time_fn(lambda: k.ce_bwd(h, W, dlogits, gs, dW, db), flush=flush)
    report("ce_bwd", ms, 2 * n * C * 2 + n * 32 * 4, rows=n)

    ids = torch.randint(4, 24, (T,), device="cuda")
    pool = torch.arange(4, 24, device="cuda", dtype=torch.int32)
    ms = time_fn(lambda: k.mlm_mask(ids, T, (0, 1, 2, 3), 3, pool, 0.3, 0.8, 0.1, 1234, 7), flush=flush)
    report("mlm_mask", ms, 3 * T * 8)

    s_t = torch.randn(T, C, device="cuda").to(BF)
    t_t = torch.randn(T, C, device="cuda").to(BF)
    valid = torch.ones(T, dtype=torch.int32, device="cuda")
    try:
        ms = time_fn(lambda: k.masked_mse(s_t, t_t, valid, torch.full((1,), 1.0 / (T * C), device="cuda")),
                     flush=flush)
        report("masked_mse", ms, 3 * T * C * 2)
    except Exception as exc:  # noqa: BLE001  (signature differences must not hide the other figures)
        print(json.dumps({"kernel": "masked_mse", "skipped": f"{type(exc).__name__}: {exc}"}), flush=True)

    # teacher attention: 32 heads of 64 channels, relative-position bias, sequences of 512
    Tb, H, D, S = min(T, 32768), 32, 64, 512
    qkv = torch.randn(Tb, 3 * H * D, device="cuda").to(BF)
    cu = torch.arange(0, Tb + 1, S, device="cuda", dtype=torch.int32)
    ss, se = k.seq_bounds(cu, Tb)
    bias_t = torch.randn(H, 2 * S - 1, device="cuda")
    ms = time_fn(lambda: k.fa_bias_fwd(qkv, ss, se, bias_t, H, D), flush=flush)
    fl = 4.0 * Tb * S * H * D
    print(json.dumps({"kernel": "fa_bias_fwd", "tokens": Tb, "heads": H, "ms": round(ms, 4),
                      "tflops": round(fl / ms / 1e9, 1)}), flush=True)

    # optimizer-step communication kernels on ONE rank: the local side of their memory traffic
    L = lib("comm")
    N = 64 * 1024 * 1024
    g = torch.randn(N, device="cuda")
    shard = torch.empty(N, device="cuda")
    sq = torch.zeros(1, device="cuda")
    one_ptr = ctypes.c_void_p * 1                          # the peer table of a single rank
    gp = one_ptr(g.data_ptr())
    ms = time_fn(lambda: L.nplm_rs_sumsq(gp, c_int(1), c_longlong(0), c_longlong(N), ptr(shard), ptr(sq),
                                         stream_ptr()))
    report("rs_sumsq (1 rank)", ms, 2 * N * 4)
    master, m, v = torch.randn(N, device="cuda"), torch.zeros(N, device="cuda"), torch.zeros(N, device="cuda")
    pb = torch.empty(N, dtype=BF, device="cuda")
    pp = one_ptr(pb.data_ptr())
    hyper = torch.tensor([1e-3, 0.9, 0.999, 1e-8, 0.0, 0.1, 0.001, 1.0, 1.0], device="cuda")
    slots = torch.ones(8, device="cuda")
    norm = torch.zeros(1, device="cuda")
    ms = time_fn(lambda: L.nplm_adamw_push(ptr(master), ptr(m), ptr(v), ptr(shard), pp, c_int(1), c_longlong(0),
                                           c_longlong(N), c_longlong(N), ptr(hyper), ptr(slots), ptr(norm),
                                           stream_ptr()))
    report("adamw_push (1 rank)", ms, N * (4 * 4 + 3 * 4 + 2))

    # Muon: momentum + Newton-Schulz input, and the parameter update, on 16 matrices of 1024 x 1024
    nmat, numel = 16, 1024 * 1024
    gm, mm = torch.randn(nmat * numel, device="cuda"), torch.zeros(nmat * numel, device="cuda")
    offs = torch.arange(nmat, device="cuda", dtype=torch.int64) * numel
    upd = torch.empty(nmat, numel, dtype=BF, device="cuda")
    usq = torch.zeros(nmat, device="cuda")
    gsq = torch.ones(1, device="cuda")
    ms = time_fn(lambda: k.muon_momentum_(gm, mm, offs, numel, upd, usq, gsq, 1.0, 1.0, 0.95, True))
    report("muon_momentum", ms, nmat * numel * (4 + 4 + 4 + 2))
    pm = torch.randn(nmat * numel, device="cuda")
    p16 = torch.empty(nmat * numel, dtype=BF, device="cuda")
    ms = time_fn(lambda: k.muon_apply_(pm, p16, offs, numel, upd, 1e-3, 0.01, True))
    report("muon_apply", ms, nmat * numel * (4 + 4 + 2 + 2))
    k.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--what", default="gemm,attn,elementwise")
    ap.add_argument("--sweep-splits", action="store_true",
                    help="gemm: time every weight-gradient shape at split-K factors 1..16 and stream-K")
    ap.add_argument("--profile", action="store_true",
                    help="launch every kernel twice only (for a profiler capture; the printed times are not bench values)")
    args = ap.parse_args()
    _PROFILE[0] = args.profile
    from nanoplm_b200.utils.peaks import measured_peaks
    peaks = measured_peaks()
    for what in args.what.split(","):
        if what == "gemm":
            bench_gemm(args.tokens, peaks, args.sweep_splits)
            continue
        {"gemm": bench_gemm, "attn": bench_attn, "attn_ws": bench_attn_ws, "elementwise": bench_elementwise, "fp8": bench_fp8,
         "moe": bench_moe, "misc": bench_misc}[what](args.tokens, peaks)


if __name__ == "__main__":
    main()
