"""Differentiable ops of the encoder.

Every op has two implementations behind one function:
  * CUDA tensors run the hand-written sm_100a kernels (``nanoplm_b200.ops.kernels``) through a
    ``torch.autograd.Function`` with an explicit backward;
  * CPU tensors run a plain fp32 PyTorch restatement. That restatement is the numerical oracle of
    the kernel tests and what the CPU plumbing configuration trains with.

Weight gradients on CUDA: when a parameter carries a ``main_grad`` attribute (fp32, a view into the
flat gradient buffer of the sharded optimizer) the weight-gradient GEMM accumulates into it
directly from its epilogue (split-K, fp32 atomics) and autograd receives no ``.grad`` for that
parameter. Without ``main_grad`` a regular gradient is returned.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import kernels as K

BF = torch.bfloat16


def _as_shape(y: torch.Tensor, shape) -> torch.Tensor:
    """y reshaped to `shape`; returns y itself (not a view object) when the shape already matches, so
    that a later in-place op on a custom Function's output stays legal for autograd."""
    shape = tuple(shape)
    return y if tuple(y.shape) == shape else y.view(shape)


def _has_main_grad(p) -> bool:
    return getattr(p, "main_grad", None) is not None


# Called with a parameter right after the kernel that adds its weight gradient into `main_grad` has
# been launched (the engine uses it to start that parameter's reduce-scatter while the rest of the
# backward pass is still running).
_WGRAD_READY = [None]


def set_wgrad_ready_callback(fn) -> None:
    _WGRAD_READY[0] = fn


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
    """dW[N,K] = dy2[T,N]^T x2[T,K]; accumulates into w.main_grad or returns a bf16 gradient."""
    T, N = dy2.shape
    Kd = x2.shape[1]
    if N % 64 == 0 and Kd % 64 == 0:
        # pair=None: single-CTA tiles unless K.set_gemm_pair_default(True). In isolation the CTA-pair
        # form is within +-5 % of them on these shapes; inside a training step both run at the rate
        # the power cap allows.
        pair = None
        if _has_main_grad(w):
            K.gemm(dy2, x2, a_mn=True, b_mn=True, epi=K.EPI_ATOMIC_F32, out=w.main_grad,
                   splits=K.wgrad_splits(N, Kd, T), pair=pair)
            if _WGRAD_READY[0] is not None:
                _WGRAD_READY[0](w)
            return None
        acc = torch.zeros((N, Kd), dtype=torch.float32, device=w.device)
        K.gemm(dy2, x2, a_mn=True, b_mn=True, epi=K.EPI_ATOMIC_F32, out=acc,
               splits=K.wgrad_splits(N, Kd, T), pair=pair)
        return acc.to(w.dtype)
    if Kd % 64 == 0 and N < 256 and dy2.is_cuda and dy2.dtype == BF and x2.dtype == BF:
        # narrow outputs (the 2n + n^2 coefficient projection of a hyper-connection site, a router):
        # pad the output columns to a whole 64 so the tensor-core kernel applies instead of an fp32
        # library GEMM over fp32 copies of both operands
        Np = (N + 63) // 64 * 64
        dyp = torch.zeros((T, Np), dtype=BF, device=dy2.device)
        dyp[:, :N] = dy2
        acc = torch.zeros((Np, Kd), dtype=torch.float32, device=w.device)
        K.gemm(dyp, x2, a_mn=True, b_mn=True, epi=K.EPI_ATOMIC_F32, out=acc, splits=K.wgrad_splits(Np, Kd, T))
        g = acc[:N]
    else:
        g = dy2.float().t() @ x2.float()
    if _has_main_grad(w):
        w.main_grad.add_(g)
        return None
    return g.to(w.dtype)


def _param_grad(p, g32: torch.Tensor):
    """Routes a small fp32 gradient (norm weights, biases) to main_grad or returns it."""
    if _has_main_grad(p):
        p.main_grad.add_(g32.view_as(p.main_grad))
        return None
    return g32.to(p.dtype).view_as(p)


# ------------------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual, act, rope=None):
        x2 = x.reshape(-1, x.shape[-1])
        if not (x2.stride(1) == 1 and x2.stride(0) % 8 == 0):
            x2 = x2.contiguous()
        pre = None
        if rope is not None:
            y = K.gemm(x2, w, epi=K.EPI_ROPE, rope=rope)
        elif act in ("gelu", "relu"):
            # the pre-activation is only kept when a backward pass will need it
            need_pre = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
            pre = torch.empty((x2.shape[0], w.shape[0]), dtype=BF, device=x.device) if need_pre else None
            y = K.gemm(x2, w, epi=K.EPI_GELU if act == "gelu" else K.EPI_RELU, aux=pre)
        elif act == "swiglu":
            pre = torch.empty((x2.shape[0], w.shape[0]), dtype=BF, device=x.device)
            y = K.gemm(x2, w, epi=K.EPI_SWIGLU, aux=pre, pair=True)   # CTA pairs: +4 % in isolation
        elif residual is not None:
            y = K.gemm(x2, w, epi=K.EPI_ADD, aux=residual.reshape(-1, w.shape[0]))
        else:
            y = K.gemm(x2, w)
        if bias is not None:
            y += bias
        ctx.save_for_backward(x2, w, pre)
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.bias_ref = bias
        ctx.x_shape = x.shape
        return _as_shape(y, (*x.shape[:-1], y.shape[1]))

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if ctx.act in ("gelu", "relu"):
            dpre = K.act_bwd(pre, dy2, ctx.act)
        elif ctx.act == "swiglu":
            dpre = K.swiglu_bwd(pre, dy2)
        else:
            dpre = dy2
        dx = None
        if ctx.needs_input_grad[0]:
            dx = _as_shape(K.gemm(dpre, w, b_mn=True), ctx.x_shape)
        dw = _wgrad(dpre, x2, w) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _param_grad(ctx.bias_ref, dpre.float().sum(0))
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres, None, None


class _SwiGLUMLPFn(torch.autograd.Function):
    """out = (silu(gate) * value) w_out^T + residual with [value | gate] = x w_in^T, as one autograd
    node so that the backward pass can compute the gradient of the pre-activations in the epilogue
    of the GEMM that produces dL/dh (no separate SwiGLU-backward pass over [T, 3I] elements)."""

    @staticmethod
    def forward(ctx, x, w_in, w_out, residual):
        x2 = x.reshape(-1, x.shape[-1])
        if not (x2.stride(1) == 1 and x2.stride(0) % 8 == 0):
            x2 = x2.contiguous()
        pre = torch.empty((x2.shape[0], w_in.shape[0]), dtype=BF, device=x.device)
        h = K.gemm(x2, w_in, epi=K.EPI_SWIGLU, aux=pre, pair=True)
        if residual is not None:
            y = K.gemm(h, w_out, epi=K.EPI_ADD, aux=residual.reshape(-1, w_out.shape[0]))
        else:
            y = K.gemm(h, w_out)
        ctx.save_for_backward(x2, w_in, w_out, pre, h)
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return _as_shape(y, (*x.shape[:-1], y.shape[1]))

    @staticmethod
    def backward(ctx, dy):
        x2, w_in, w_out, pre, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dpre = K.gemm(dy2, w_out, b_mn=True, epi=K.EPI_SWIGLU_BWD, aux=pre)
        dw_out = _wgrad(dy2, h, w_out) if ctx.needs_input_grad[2] else None
        dw_in = _wgrad(dpre, x2, w_in) if ctx.needs_input_grad[1] else None
        dx = _as_shape(K.gemm(dpre, w_in, b_mn=True), ctx.x_shape) if ctx.needs_input_grad[0] else None
        return dx, dw_in, dw_out, (dy if ctx.has_res else None)


def mlp_swiglu(x, w_in, w_out, residual=None):
    """SwiGLU MLP block (w_in rows = [value | gate]) + residual. CUDA bf16 with 64-aligned widths:
    one autograd node with the fused backward epilogue; otherwise two `linear` calls."""
    inter = w_out.shape[1]
    if (x.is_cuda and x.dtype == BF and not _FP8_STATE["enabled"] and inter % 64 == 0 and w_in.shape[0] == 2 * inter
            and w_in.shape[1] % 64 == 0 and w_out.shape[0] % 64 == 0):
        return _SwiGLUMLPFn.apply(x, w_in, w_out, residual)
    return linear(linear(x, w_in, act="swiglu"), w_out, residual=residual)


def linear_rope(x, w, pos, cos, sin, rope_cols: int):
    """QKV projection with the rotary embedding of q and k applied in the GEMM epilogue (CUDA,
    head_dim 64). The result equals rope_qkv(linear(x, w)); its gradient w.r.t. the un-rotated
    projection is obtained by passing rope=(pos, cos, sin) to attention_varlen."""
    return _LinearFn.apply(x, w, None, None, None, (pos, cos, sin, rope_cols))


_FP8_STATE = {"enabled": False}


def set_fp8(enabled: bool) -> None:
    """Routes every bias-free linear layer whose weight dims are multiples of 128 through the
    e4m3 block-scaled GEMM (forward, data gradient and weight gradient); see nanoplm_b200.ops.fp8.
    The reference has no FP8 mode."""
    _FP8_STATE["enabled"] = bool(enabled)


def fp8_enabled() -> bool:
    return _FP8_STATE["enabled"]


def linear(x, w, bias=None, residual=None, act: str | None = None):
    """y = act(x w^T + bias) + residual.  act: None | "gelu" | "relu" | "swiglu" (w rows = [value | gate],
    output is half as wide). residual and act are mutually exclusive."""
    if x.is_cuda and _FP8_STATE["enabled"] and bias is None:
        from . import fp8
        if fp8.supported(x, w):
            y = fp8.fp8_linear(x, w)
            if act == "swiglu":
                y = swiglu(y)
            elif act in ("gelu", "relu"):
                y = activation(y, act)
            if residual is not None:
                y = y + residual
            return y
    if x.is_cuda:
        if w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.dtype == BF:
            if act == "swiglu" and bias is not None:
                y = _LinearFn.apply(x, w, bias, None, None)
                return swiglu(y)
            return _LinearFn.apply(x, w, bias, residual, act)
    y = F.linear(x, w, bias)
    if act == "gelu":
        y = F.gelu(y)
    elif act == "relu":
        y = F.relu(y)
    elif act == "swiglu":
        v, g = y.chunk(2, dim=-1)
        y = F.silu(g) * v
    if residual is not None:
        y = y + residual
    return y


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre):
        p2 = pre.reshape(-1, pre.shape[-1]).contiguous()
        ctx.save_for_backward(p2)
        ctx.shape = pre.shape
        return _as_shape(K.swiglu_fwd(p2), (*pre.shape[:-1], pre.shape[-1] // 2))

    @staticmethod
    def backward(ctx, dy):
        (p2,) = ctx.saved_tensors
        return _as_shape(K.swiglu_bwd(p2, dy.reshape(-1, dy.shape[-1]).contiguous()), ctx.shape)


def swiglu(pre):
    """pre = [value | gate] -> silu(gate) * value (reference: modeling.py:301-302)."""
    if pre.is_cuda and pre.dtype == BF:
        return _SwigluFn.apply(pre)
    v, g = pre.chunk(2, dim=-1)
    return F.silu(g) * v


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre, name):
        p = pre.contiguous()
        ctx.save_for_backward(p)
        ctx.name = name
        return K.act_fwd(p, name)

    @staticmethod
    def backward(ctx, dy):
        (p,) = ctx.saved_tensors
        return K.act_bwd(p, dy.contiguous(), ctx.name), None


def activation(x, name: str):
    if x.is_cuda and x.dtype == BF and x.numel() % 8 == 0 and name in ("gelu", "relu", "silu"):
        return _ActFn.apply(x, name)
    return {"gelu": F.gelu, "relu": F.relu, "silu": F.silu, "tanh": torch.tanh}[name](x)


# ------------------------------------------------------------------------------------- norms
class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, rms):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, mean, rstd = K.norm_fwd(x2, w, eps, rms=rms)
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.rms = rms
        ctx.shape = x.shape
        return _as_shape(y, x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        dw = None
        if w is not None and ctx.needs_input_grad[1]:
            dw = w.main_grad if _has_main_grad(w) else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dx = K.norm_bwd(dy, x2, w, mean, rstd, rms=ctx.rms, dw=dw)
        if dw is not None:
            dw = None if _has_main_grad(w) else dw.to(w.dtype)
        return _as_shape(dx, ctx.shape), dw, None, None


class _NormResFn(torch.autograd.Function):
    """norm(x) plus x itself as a second output. In a pre-norm residual block both the branch and
    the skip connection start at x; routing the skip through this function lets the backward add
    the skip gradient inside the norm-backward kernel instead of a separate elementwise pass."""

    @staticmethod
    def forward(ctx, x, w, eps, rms):
        x2 = x if x.is_contiguous() else x.contiguous()
        y, mean, rstd = K.norm_fwd(x2, w, eps, rms=rms)
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.rms = rms
        return y, x2.view_as(x2)

    @staticmethod
    def backward(ctx, dy, dres):
        x2, w, mean, rstd = ctx.saved_tensors
        dw = None
        if w is not None and ctx.needs_input_grad[1]:
            dw = w.main_grad if _has_main_grad(w) else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        if dy is None:
            return dres, None, None, None
        if dres is not None and not dres.is_contiguous():
            dres = dres.contiguous()
        dx = K.norm_bwd(dy, x2, w, mean, rstd, rms=ctx.rms, dres=dres, dw=dw)
        if dw is not None:
            dw = None if _has_main_grad(w) else dw.to(w.dtype)
        return dx, dw, None, None


def norm_residual(x, w, eps: float = 1e-5, rms: bool = False):
    """Returns (norm(x), x) — see _NormResFn. x is a flat [T, C] activation."""
    if x.is_cuda and x.dtype == BF and x.dim() == 2 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096:
        return _NormResFn.apply(x, w, eps, rms)
    return norm(x, w, eps, rms), x


def norm(x, w, eps: float = 1e-5, rms: bool = False):
    """LayerNorm without bias (reference encoder norms) or RMSNorm (T5LayerNorm) over the last dim."""
    if x.is_cuda and x.dtype == BF and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096:
        return _NormFn.apply(x, w, eps, rms)
    xf = x.float()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            y = y * w.float()
    else:
        y = F.layer_norm(xf, (x.shape[-1],), None if w is None else w.float(), None, eps)
    return y.to(x.dtype)


class _EmbedNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, w, eps, rms):
        ids32 = ids.to(torch.int32).contiguous()
        y, mean, rstd = K.norm_fwd(table, w, eps, rms=rms, ids=ids32)
        ctx.save_for_backward(ids32, table, w, mean, rstd)
        ctx.rms = rms
        return y

    @staticmethod
    def backward(ctx, dy):
        ids32, table, w, mean, rstd = ctx.saved_tensors
        dt = table.main_grad if _has_main_grad(table) else torch.zeros(table.shape, dtype=torch.float32,
                                                                      device=table.device)
        dw = w.main_grad if _has_main_grad(w) else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        K.norm_bwd(dy, table, w, mean, rstd, rms=ctx.rms, ids=ids32, dtable=dt, dw=dw)
        return (None, None if _has_main_grad(table) else dt.to(table.dtype),
                None if _has_main_grad(w) else dw.to(w.dtype), None, None)


def embed_norm(ids, table, w, eps: float = 1e-5, rms: bool = False):
    """norm(table[ids]) for flat ids (reference: modeling.py:222-223)."""
    if table.is_cuda and table.dtype == BF and table.shape[1] % 8 == 0 and table.shape[1] <= 4096:
        return _EmbedNormFn.apply(ids, table, w, eps, rms)
    return norm(F.embedding(ids.long(), table), w, eps, rms)


# ------------------------------------------------------------------------------------- rope
def rope_tables(max_pos: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [max_pos, head_dim/2] fp32 (the reference table is these halves repeated twice,
    modeling.py:241-261)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    fr = torch.outer(torch.arange(max_pos, dtype=torch.float32, device=device), inv)
    return fr.cos().contiguous(), fr.sin().contiguous()


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, pos, cos, sin, H, D):
        ctx.save_for_backward(pos, cos, sin)
        ctx.hd = (H, D)
        K.rope_(qkv, pos, cos, sin, H, D)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, d):
        pos, cos, sin = ctx.saved_tensors
        d = d.contiguous()
        K.rope_(d, pos, cos, sin, *ctx.hd, backward=True)
        return d, None, None, None, None, None


def rope_qkv(qkv, pos, cos, sin, H: int, D: int):
    """Rotates the q and k parts of qkv [T, 3*H*D] (rotate-half convention, fp32 math)."""
    if qkv.is_cuda and qkv.dtype == BF and D % 16 == 0:
        return _RopeFn.apply(qkv, pos, cos, sin, H, D)
    T = qkv.shape[0]
    x = qkv.view(T, 3, H, D)
    c = torch.cat((cos, cos), -1)[pos.long()][:, None, :]
    s = torch.cat((sin, sin), -1)[pos.long()][:, None, :]

    def rot(t):
        tf = t.float()
        t1, t2 = tf.chunk(2, dim=-1)
        return (tf * c + torch.cat((-t2, t1), -1) * s).to(t.dtype)

    return torch.stack((rot(x[:, 0]), rot(x[:, 1]), x[:, 2]), dim=1).reshape(T, 3 * H * D)


# ------------------------------------------------------------------------------------- attention
class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, seq_start, seq_end, H, D, window, scale, rope):
        out, lse = K.fa_fwd(qkv, seq_start, seq_end, H, D, window, scale)
        ctx.save_for_backward(qkv, out, lse, seq_start, seq_end)
        ctx.cfg = (H, D, window, scale)
        ctx.rope = rope
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, ss, se = ctx.saved_tensors
        H, D, window, scale = ctx.cfg
        dqkv = K.fa_bwd(qkv, out, dout.contiguous(), lse, ss, se, H, D, window, scale, rope=ctx.rope)
        return dqkv, None, None, None, None, None, None, None


class _AttnOutFn(torch.autograd.Function):
    """Attention followed by its output projection (+ residual) as one autograd node: the GEMM that
    turns dy into dO also emits rowsum(dO * O) from its epilogue, so the attention backward does
    not read O and dO once more for it."""

    @staticmethod
    def forward(ctx, qkv, w_out, residual, seq_start, seq_end, H, D, window, scale, rope):
        out, lse = K.fa_fwd(qkv, seq_start, seq_end, H, D, window, scale)
        if residual is not None:
            y = K.gemm(out, w_out, epi=K.EPI_ADD, aux=residual.reshape(-1, w_out.shape[0]))
        else:
            y = K.gemm(out, w_out)
        ctx.save_for_backward(qkv, out, lse, seq_start, seq_end, w_out)
        ctx.cfg = (H, D, window, scale)
        ctx.rope = rope
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        qkv, out, lse, ss, se, w_out = ctx.saved_tensors
        H, D, window, scale = ctx.cfg
        dy2 = dy if dy.is_contiguous() else dy.contiguous()
        delta = torch.empty((H, qkv.shape[0]), dtype=torch.float32, device=qkv.device)
        dout = K.gemm_dgrad_delta(dy2, w_out, out, delta)
        dw = _wgrad(dy2, out, w_out) if ctx.needs_input_grad[1] else None
        dqkv = K.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale, delta=delta, rope=ctx.rope,
                        delta_ready=True)
        return dqkv, dw, (dy if ctx.has_res else None), None, None, None, None, None, None, None


def attention_out_proj(qkv, w_out, residual, seq_start, seq_end, H: int, D: int, window: int, scale: float,
                       rope=None):
    """attention_varlen(qkv, ...) @ w_out^T + residual. CUDA bf16, head_dim 64, 2-D activations and a
    bias-free projection run as one autograd node (fused backward); otherwise the two separate ops."""
    if (qkv.is_cuda and qkv.dtype == BF and D == 64 and qkv.dim() == 2 and not _FP8_STATE["enabled"]
            and w_out.shape[1] == H * D and w_out.shape[0] % 8 == 0):
        return _AttnOutFn.apply(qkv, w_out, residual, seq_start, seq_end, H, D, window, scale, rope)
    return linear(attention_varlen(qkv, seq_start, seq_end, H, D, window, scale, rope=rope), w_out,
                  residual=residual)


def seq_bounds(cu_seqlens: torch.Tensor, T: int):
    """Per-token [start, end) of the sequence each flat token belongs to."""
    if cu_seqlens.is_cuda:
        return K.seq_bounds(cu_seqlens.to(torch.int32), T)
    cu = cu_seqlens.long()
    t = torch.arange(T)
    idx = torch.searchsorted(cu, t, right=True) - 1
    idx = idx.clamp(0, len(cu) - 2)
    a, b = cu[idx], cu[idx + 1]
    bad = (t < a) | (t >= b)
    a = torch.where(bad, t, a)
    b = torch.where(bad, t + 1, b)
    return a.to(torch.int32), b.to(torch.int32)


def attention_varlen(qkv, seq_start, seq_end, H: int, D: int, window: int, scale: float, rope=None):
    """Non-causal attention inside each packed sequence; window >= 0 limits |q - k| <= window.
    rope=(pos, cos, sin) (CUDA only) declares that q / k were rotated by linear_rope: the backward
    then returns the gradient of the un-rotated projection."""
    if qkv.is_cuda and qkv.dtype == BF and D == 64:
        return _AttnFn.apply(qkv, seq_start, seq_end, H, D, window, scale, rope)
    if rope is not None:
        raise ValueError("fused rope backward is only available on the CUDA kernels")
    T = qkv.shape[0]
    q, k, v = qkv.view(T, 3, H, D).unbind(1)
    pos = torch.arange(T, device=qkv.device)
    mask = (pos[None, :] >= seq_start.long()[:, None]) & (pos[None, :] < seq_end.long()[:, None])
    if window >= 0:
        mask &= (pos[:, None] - pos[None, :]).abs() <= window
    s = torch.einsum("thd,shd->hts", q.float(), k.float()) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, v.float()).reshape(T, H * D).to(qkv.dtype)


# ------------------------------------------------------------------------------------- gather
class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx):
        ctx.save_for_backward(idx)
        ctx.rows = x.shape[0]
        return K.gather_rows(x, idx)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        dx = torch.zeros((ctx.rows, dy.shape[1]), dtype=dy.dtype, device=dy.device)
        K.scatter_rows_(dx, idx, dy.contiguous())
        return dx, None


def gather_rows(x, idx):
    """x[idx] for unique row indices (int32)."""
    if x.is_cuda and x.dtype == BF and x.shape[1] % 8 == 0:
        return _GatherFn.apply(x.contiguous(), idx.to(torch.int32))
    return x[idx.long()]


# ------------------------------------------------------------------------------------- loss
class _CEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, W, bias, labels, want_logits):
        n_valid = (labels >= 0).sum().clamp(min=1).float()
        inv = (1.0 / n_valid).reshape(1)
        loss, dlogits, logits = K.ce_fwd(h, W, bias, labels, inv, want_logits)
        ctx.save_for_backward(h, W, dlogits)
        ctx.bias_ref = bias
        ctx.w_ref = W
        ctx.mark_non_differentiable(*([logits] if logits is not None else []))
        if logits is None:
            logits = torch.empty(0, device=h.device)
        return loss.squeeze(0), logits

    @staticmethod
    def backward(ctx, dloss, _dlogits):
        h, W, dlogits = ctx.saved_tensors
        bias = ctx.bias_ref
        V = W.shape[0]
        dW = W.main_grad if _has_main_grad(W) else torch.zeros(W.shape, dtype=torch.float32, device=W.device)
        db = None
        if bias is not None:
            db = bias.main_grad if _has_main_grad(bias) else torch.zeros(V, dtype=torch.float32, device=W.device)
        gs = dloss.float().reshape(1).contiguous()
        dh = K.ce_bwd(h, W, dlogits, gs, dW, db)
        gW = None if _has_main_grad(W) else dW.to(W.dtype)
        gb = None
        if bias is not None:
            gb = None if _has_main_grad(bias) else db.to(bias.dtype)
        return dh, gW, gb, None, None


def mlm_cross_entropy(h, W, bias, labels, want_logits: bool = False):
    """mean_{labels != -100} CE(h W^T + bias, labels). Returns (loss, logits or None).

    Fused kernel for vocabularies of at most 32 entries (decoder GEMM, log-sum-exp, loss and
    dlogits in one pass; reference: modeling.py:659-664)."""
    if h.is_cuda and h.dtype == BF and W.shape[0] <= 32 and h.shape[1] % 8 == 0 and h.shape[1] <= 4096:
        loss, logits = _CEFn.apply(h.contiguous(), W, bias, labels.to(torch.int32).contiguous(), want_logits)
        return loss, (logits if want_logits else None)
    logits = F.linear(h, W, bias)
    loss = F.cross_entropy(logits.float(), labels.long(), ignore_index=-100)
    return loss, (logits if want_logits else None)


class _MSEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s, t, valid):
        v32 = None if valid is None else valid.to(torch.int32).contiguous()
        n = (v32.sum() if v32 is not None else torch.tensor(s.shape[0], device=s.device)).clamp(min=1).float()
        inv = (1.0 / n).reshape(1)
        loss, ds = K.masked_mse(s, t, v32, inv, want_grad=True)
        ctx.save_for_backward(ds)
        return loss.squeeze(0)

    @staticmethod
    def backward(ctx, dloss):
        (ds,) = ctx.saved_tensors
        return ds * dloss.to(ds.dtype), None, None


def masked_mse(student, teacher, valid=None):
    """sum over features, mean over valid tokens of (student - teacher)^2
    (reference: src/nanoplm/distillation/trainer.py:30-40). Inputs are [T, C]."""
    if student.is_cuda and student.dtype == BF and student.shape[1] % 8 == 0:
        return _MSEFn.apply(student.contiguous(), teacher.to(BF).contiguous(), valid)
    d = (student.float() - teacher.float()) ** 2
    if valid is not None:
        m = valid.to(d.dtype)[:, None]
        return (d * m).sum() / m.sum().clamp(min=1)
    return d.sum() / max(1, student.shape[0])
