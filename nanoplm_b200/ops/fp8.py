"""FP8 (e4m3) block-scaled linear layers: quantisation kernels, the tcgen05 fp8 GEMM with
per-128-K-block promotion (nanoplm_b200/csrc/fp8.cu) and the autograd function that runs forward,
data gradient and weight gradient on e4m3 operands.

Recipe ("block128"): activations and gradients are scaled per 1 x 128 along the contraction axis
of the GEMM that consumes them, weights per 128 x 128; accumulation is fp32; master weights stay
bf16 / fp32 in the optimizer. The reference has no FP8 path (it trains under a bf16
MixedPrecisionPolicy, src/nanoplm/pretraining/pure_pipeline.py:485-487).

Quantised weights are cached per parameter and re-used across the micro-steps of one optimizer
step; `invalidate_weight_cache()` is called by the engines after every parameter update.
"""
from __future__ import annotations

from ctypes import c_int

import torch

from ._lib import check_rc, count_launch, lib, ptr, status_word, stream_ptr

_BF16 = torch.bfloat16
E4M3_MAX = 448.0


class Quantized:
    """e4m3 payload (uint8 view) [rows, K] with fp32 scales stored K-block-major."""
    __slots__ = ("q", "scale", "block")

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, block: bool):
        self.q, self.scale, self.block = q, scale, block

    def dequantize(self) -> torch.Tensor:
        """fp32 tensor of the represented values (test helper)."""
        rows, K = self.q.shape
        v = self.q.view(torch.float8_e4m3fn).float()
        if self.block:
            s = self.scale.view(K // 128, -1)                     # [KB, row blocks]
            s = s.repeat_interleave(128, dim=1)[:, :rows]          # [KB, rows]
        else:
            s = self.scale.view(K // 128, rows)
        return v * s.t().repeat_interleave(128, dim=1)


def quant_rows(x: torch.Tensor) -> Quantized:
    """x bf16 [R, K] (K % 128 == 0) -> e4m3 with 1 x 128 scales along K."""
    R, K = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    q = torch.empty((R, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((K // 128, R), dtype=torch.float32, device=x.device)
    rc = lib("fp8").nplm_fp8_quant_rows(ptr(x), c_int(R), c_int(K), c_int(x.stride(0)), ptr(q), ptr(s), stream_ptr())
    check_rc(rc, "fp8_quant_rows")
    count_launch()
    return Quantized(q, s, False)


def quant_tile(x: torch.Tensor, transpose: bool, block: bool) -> Quantized:
    """128 x 128 tile quantisation of x bf16 [R, K].

    transpose=False, block=True : payload [R, K], one scale per 128 x 128 tile (weights)
    transpose=True,  block=True : payload [K, R] (weights for the data-gradient GEMM)
    transpose=True,  block=False: payload [K, R] with 1 x 128 scales along R (operands of the
                                  weight-gradient GEMM, which contracts over tokens)
    """
    R, K = x.shape
    if x.stride(1) != 1:
        x = x.contiguous()
    if transpose:
        q = torch.empty((K, R), dtype=torch.uint8, device=x.device)
        rb = (R + 127) // 128
        s = torch.empty((rb, K // 128) if block else (rb, K), dtype=torch.float32, device=x.device)
    else:
        q = torch.empty((R, K), dtype=torch.uint8, device=x.device)
        s = torch.empty((K // 128, R // 128), dtype=torch.float32, device=x.device)
    rc = lib("fp8").nplm_fp8_quant_tile(ptr(x), c_int(R), c_int(K), c_int(x.stride(0)), c_int(int(transpose)),
                                        c_int(int(block)), ptr(q), ptr(s), stream_ptr())
    check_rc(rc, "fp8_quant_tile")
    count_launch()
    return Quantized(q, s, block)


def gemm_fp8(a: Quantized, b: Quantized, *, out: torch.Tensor | None = None, out_dtype=_BF16,
             accumulate: bool = False) -> torch.Tensor:
    """C[M,N] (+)= deq(a) deq(b)^T. a: row-scaled [M,K]; b: row- or block-scaled [N,K]."""
    if a.block:
        raise ValueError("the A operand must carry 1 x 128 scales")
    M, K = a.q.shape
    N, Kb = b.q.shape
    if K != Kb:
        raise ValueError(f"inner dims differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an fp32 out tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.q.device)
    mode = 0 if out.dtype == _BF16 else (2 if accumulate else 1)
    if out.dtype not in (_BF16, torch.float32) or tuple(out.shape) != (M, N) or out.stride(1) != 1:
        raise ValueError("out must be a row-major bf16 or fp32 [M, N] tensor")
    rc = lib("fp8").nplm_gemm_fp8(ptr(a.q), ptr(b.q), ptr(out), ptr(a.scale), ptr(b.scale), c_int(M), c_int(N),
                                  c_int(K), c_int(out.stride(0)), c_int(int(b.block)), c_int(mode),
                                  ptr(status_word(a.q.device)), stream_ptr())
    check_rc(rc, "gemm_fp8")
    count_launch()
    return out


def gemm_fp8_ag(a: Quantized, b_payload: torch.Tensor, b_payload_ptrs, b_scale: torch.Tensor, b_scale_ptrs,
                rank: int, world: int, flags: torch.Tensor, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather fused into the fp8 GEMM: C = deq(a) deq(B)^T with B's rows (e4m3 payload [N,K] and
    block scales [K/128, N/128]) sharded over `world` ranks in peer-mapped memory. b_payload /
    b_scale are this rank's full-size buffers (only its shard valid on entry, everything valid on
    return); *_ptrs are the ctypes arrays of every rank's buffer addresses. The fp8 payload moves
    half the bytes of a bf16 gather. flags: int32 [8]."""
    M, K = a.q.shape
    N = b_payload.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=_BF16, device=a.q.device)
    mode = 0 if out.dtype == _BF16 else 1
    rc = lib("fp8").nplm_gemm_fp8_ag(ptr(a.q), b_payload_ptrs, ptr(out), ptr(a.scale), b_scale_ptrs, c_int(M),
                                     c_int(N), c_int(K), c_int(out.stride(0)), c_int(mode), c_int(rank),
                                     c_int(world), ptr(flags), ptr(status_word(a.q.device)), stream_ptr())
    check_rc(rc, "gemm_fp8_ag")
    count_launch()
    return out


# ------------------------------------------------------------------------------ weight cache
_weight_cache: dict[int, tuple] = {}


def invalidate_weight_cache() -> None:
    _weight_cache.clear()


def _quantized_weight(w: torch.Tensor):
    """(W as [N,K] block-scaled, W^T as [K,N] block-scaled) for this parameter version."""
    key = id(w)
    hit = _weight_cache.get(key)
    if hit is not None and hit[0] == w.data_ptr():
        return hit[1], hit[2]
    qw = quant_tile(w.detach(), transpose=False, block=True)
    qwt = quant_tile(w.detach(), transpose=True, block=True)
    _weight_cache[key] = (w.data_ptr(), qw, qwt)
    return qw, qwt


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the fp8 path covers: bf16 CUDA tensors, both weight dims multiples of 128."""
    return (x.is_cuda and x.dtype == _BF16 and w.dtype == _BF16 and w.shape[0] % 128 == 0
            and w.shape[1] % 128 == 0)


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        from .functional import _as_shape
        x2 = x.reshape(-1, x.shape[-1])
        qx = quant_rows(x2)
        qw, _ = _quantized_weight(w)
        y = gemm_fp8(qx, qw)
        ctx.save_for_backward(x2, w)
        ctx.w_ref = w
        ctx.shape = x.shape
        return _as_shape(y, (*x.shape[:-1], w.shape[0]))

    @staticmethod
    def backward(ctx, dy):
        from .functional import _as_shape, _has_main_grad, _wgrad
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            _, qwt = _quantized_weight(ctx.w_ref)
            dx = _as_shape(gemm_fp8(quant_rows(dy2), qwt), ctx.shape)
        if ctx.needs_input_grad[1]:
            T = x2.shape[0]
            if T % 128 == 0:
                # dW[N,K] = dY^T X: both operands transposed to token-contiguous payloads
                qdy_t = quant_tile(dy2, transpose=True, block=False)
                qx_t = quant_tile(x2, transpose=True, block=False)
                p = ctx.w_ref
                if _has_main_grad(p):
                    gemm_fp8(qdy_t, qx_t, out=p.main_grad.view(w.shape), accumulate=True)
                else:
                    dw = gemm_fp8(qdy_t, qx_t, out_dtype=torch.float32).to(w.dtype)
            else:
                dw = _wgrad(dy2, x2, ctx.w_ref)
        return dx, dw


def fp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x W^T with e4m3 operands (no bias)."""
    return _Fp8LinearFn.apply(x, w)
