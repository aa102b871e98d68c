"""Varlen depthwise convolution block (kernel 7 by default), applied to the normed block input
before attention and added back residually. Taps never cross a sequence boundary of the packed
batch: positions outside `[seq_start, seq_end)` of the token's own sequence contribute zero.
The reference has no such block; semantics are documented in nanoplm_b200/csrc/extras.cu."""
from __future__ import annotations

import torch
import torch.nn as nn

from nanoplm_b200.ops import kernels as K
from nanoplm_b200.ops.functional import _has_main_grad


def dwconv_reference(x, w, bias, seq_start, seq_end):
    """fp32 restatement: y[t,c] = bias[c] + sum_k w[c,k] x[t+k-r,c] [same sequence]."""
    T, C = x.shape
    KS = w.shape[1]
    r = KS // 2
    t = torch.arange(T, device=x.device)
    y = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    xf = x.float()
    for k in range(KS):
        src = t + (k - r)
        ok = (src >= seq_start.long()) & (src < seq_end.long())
        src = src.clamp(0, T - 1)
        y = y + torch.where(ok[:, None], xf[src], torch.zeros_like(xf)) * w.float()[:, k][None, :]
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


class _DWConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ss, se):
        x = x.contiguous()
        ctx.save_for_backward(x, w, ss, se)
        ctx.bias_ref = bias
        ctx.w_ref = w
        return K.dwconv(x, w.contiguous(), bias, ss, se)

    @staticmethod
    def backward(ctx, dy):
        x, w, ss, se = ctx.saved_tensors
        dy = dy.contiguous()
        dx = K.dwconv(dy, w.contiguous(), None, ss, se, flip=True)
        bias = ctx.bias_ref
        dw = w.main_grad if _has_main_grad(w) else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        db = None
        if bias is not None:
            db = bias.main_grad if _has_main_grad(bias) else torch.zeros(bias.shape, dtype=torch.float32, device=w.device)
        K.dwconv_bwd_w(x, dy, ss, se, dw, db)
        gw = None if _has_main_grad(w) else dw.to(w.dtype)
        gb = None if (bias is None or _has_main_grad(bias)) else db.to(bias.dtype)
        return dx, gw, gb, None, None


def dwconv_varlen(x, w, bias, seq_start, seq_end):
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.shape[1] <= 9:
        return _DWConvFn.apply(x, w, bias, seq_start, seq_end)
    return dwconv_reference(x, w, bias, seq_start, seq_end)


class VarlenDepthwiseConv(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 7, bias: bool = False):
        super().__init__()
        self.kernel_size = kernel_size
        w = torch.zeros(channels, kernel_size)
        nn.init.normal_(w, 0.0, 0.02)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(channels)) if bias else None

    def forward(self, x, ctx):
        return dwconv_varlen(x, self.weight, self.bias, ctx.seq_start, ctx.seq_end)
