"""Manifold-constrained hyper-connections (mHC): n parallel residual streams X[T, n, C].

Per sub-layer (attention or MLP) and per token:
    z      = rmsnorm(mean_i X_i)                                  (what the coefficient net sees)
    alpha  = softmax(a + s_a * tanh(W_a z))            [n]        read weights
    beta   = 2 * sigmoid(b + s_b * tanh(W_b z))        [n]        write weights
    R      = sinkhorn(exp(r + s_r * tanh(W_r z)))      [n, n]     residual mixing, projected onto the
                                                                  doubly-stochastic matrices (the
                                                                  "manifold constraint")
    h      = sum_i alpha_i X_i                         read
    X_i   <- sum_j R_ij X_j + beta_i f(h)              write
Static parts start at the plain-residual solution (alpha uniform, beta = 1, R = identity) and the
dynamic scales s_* start at 0.01, so a fresh model behaves like an ordinary pre-norm residual
network whose streams are n copies of the embedding; the streams are summed before the final norm.
The reference has no hyper-connections; the stream mixing runs in nanoplm_b200/csrc/extras.cu.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanoplm_b200.ops import kernels as K


def sinkhorn(logits: torch.Tensor, iters: int) -> torch.Tensor:
    """Projects exp(logits) [..., n, n] towards a doubly-stochastic matrix (log-domain Sinkhorn)."""
    x = logits
    for _ in range(max(1, iters)):
        x = x - torch.logsumexp(x, dim=-1, keepdim=True)
        x = x - torch.logsumexp(x, dim=-2, keepdim=True)
    return x.exp()


class _ReadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, alpha):
        X = X.contiguous()
        alpha = alpha.float().contiguous()
        ctx.save_for_backward(X, alpha)
        return K.mhc_read(X, alpha)

    @staticmethod
    def backward(ctx, dh):
        X, alpha = ctx.saved_tensors
        dX, _, _, dalpha, _ = K.mhc_bwd(X, None, None, alpha, None, None, dh.contiguous())
        return dX, dalpha


class _WriteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, y, R, beta):
        X, y = X.contiguous(), y.contiguous()
        R, beta = R.float().contiguous(), beta.float().contiguous()
        ctx.save_for_backward(X, y, R, beta)
        return K.mhc_write(X, y, R, beta)

    @staticmethod
    def backward(ctx, dXn):
        X, y, R, beta = ctx.saved_tensors
        dX, dy, dR, _, dbeta = K.mhc_bwd(X, y, R, None, beta, dXn.contiguous(), None)
        return dX, dy, dR, dbeta


class _SiteGrad:
    """Hand-over between the two backward nodes of one site (see _MeanFn)."""
    __slots__ = ("alpha", "dh")

    def __init__(self):
        self.alpha = self.dh = None


class _MeanFn(torch.autograd.Function):
    """z = stream mean of X, and X itself handed on as X1 for the read and the write of the site.

    The streams entering a site have three consumers (the mean for the coefficient network, the
    read and the write); left to autograd that is three [T, n, C] gradients and two sums. Here X is
    threaded through the site instead (X -> X1 -> read -> X2 -> write), the read's backward only
    computes d alpha and leaves (alpha, dh) in `site`, and this node, which runs last, forms
    dX = dX2 + alpha dh + dz / n in one pass."""

    @staticmethod
    def forward(ctx, X, site):
        ctx.site = site
        ctx.shape = tuple(X.shape)
        return K.mhc_mean(X), X.view_as(X)

    @staticmethod
    def backward(ctx, dz, g):
        site = ctx.site
        alpha, dh = site.alpha, site.dh
        site.alpha = site.dh = None
        dz = dz.contiguous() if dz is not None else None
        g = g.contiguous() if g is not None else None
        if g is None and dh is None and dz is None:
            return None, None
        return K.mhc_dx_combine(g, alpha, dh, dz, ctx.shape), None


class _ReadThreadFn(torch.autograd.Function):
    """h = sum_i alpha_i X1_i, and X1 handed on as X2 for the write. Backward: d alpha only; the
    gradient arriving for X2 goes back unchanged and _MeanFn adds the read's share to it."""

    @staticmethod
    def forward(ctx, X1, alpha, site):
        alpha = alpha.float().contiguous()
        ctx.save_for_backward(X1, alpha)
        ctx.site = site
        return K.mhc_read(X1, alpha), X1.view_as(X1)

    @staticmethod
    def backward(ctx, dh, g):
        X1, alpha = ctx.saved_tensors
        dalpha = None
        if dh is not None:
            dh = dh.contiguous()
            _, _, _, dalpha, _ = K.mhc_bwd(X1, None, None, alpha, None, None, dh, want_dx=False)
            ctx.site.alpha, ctx.site.dh = alpha, dh
        return g, dalpha, None


def mhc_read(X, alpha):
    if X.is_cuda and X.dtype == torch.bfloat16 and X.shape[-1] % 8 == 0 and X.shape[1] <= 4:
        return _ReadFn.apply(X, alpha)
    return torch.einsum("ti,tic->tc", alpha.to(X.dtype), X)


def mhc_write(X, y, R, beta):
    if X.is_cuda and X.dtype == torch.bfloat16 and X.shape[-1] % 8 == 0 and X.shape[1] <= 4:
        return _WriteFn.apply(X, y, R, beta)
    return torch.einsum("tij,tjc->tic", R.to(X.dtype), X) + beta.to(X.dtype)[:, :, None] * y[:, None, :]


class _CoefFn(torch.autograd.Function):
    """(raw projections, static parts, scales) -> (alpha, beta, R) in one kernel each way
    (tanh, softmax, sigmoid and the log-domain Sinkhorn iterations; nanoplm_b200/csrc/extras.cu)."""

    @staticmethod
    def forward(ctx, pre, a, b, r, s, iters, n):
        pre = pre.contiguous()
        a32, b32, r32, s32 = (t.detach().float().contiguous() for t in (a, b, r, s))
        alpha, beta, R = K.mhc_coef_fwd(pre, a32, b32, r32, s32, iters, n)
        ctx.save_for_backward(pre, a32, b32, r32, s32)
        ctx.iters, ctx.n = iters, n
        ctx.refs = (a, b, r, s)
        return alpha, beta, R

    @staticmethod
    def backward(ctx, dalpha, dbeta, dR):
        from nanoplm_b200.ops.functional import _param_grad
        pre, a32, b32, r32, s32 = ctx.saved_tensors
        n, dev = ctx.n, pre.device
        T = pre.shape[0]
        zeros = lambda *shape: torch.zeros(shape, dtype=torch.float32, device=dev)
        dalpha = dalpha.float().contiguous() if dalpha is not None else zeros(T, n)
        dbeta = dbeta.float().contiguous() if dbeta is not None else zeros(T, n)
        dR = dR.float().contiguous() if dR is not None else zeros(T, n, n)
        da, db, dr, ds = zeros(n), zeros(n), zeros(n, n), zeros(3)
        dpre = K.mhc_coef_bwd(pre, a32, b32, r32, s32, ctx.iters, n, dalpha, dbeta, dR, da, db, dr, ds)
        a, b, r, s = ctx.refs
        return dpre, _param_grad(a, da), _param_grad(b, db), _param_grad(r, dr), _param_grad(s, ds), None, None


class HyperConnection(nn.Module):
    def __init__(self, dim: int, n: int, sinkhorn_iters: int = 5, eps: float = 1e-5):
        super().__init__()
        self.n, self.iters, self.eps = n, sinkhorn_iters, eps
        self.coef_norm_weight = nn.Parameter(torch.ones(dim))
        self.coef_proj = nn.Linear(dim, 2 * n + n * n, bias=False)
        nn.init.normal_(self.coef_proj.weight, 0.0, 0.02)
        self.static_alpha = nn.Parameter(torch.zeros(n))
        self.static_beta = nn.Parameter(torch.zeros(n))            # 2*sigmoid(0) = 1
        self.static_res = nn.Parameter(torch.eye(n) * 6.0 - 3.0)   # sinkhorn(exp(.)) ~ identity
        self.dyn_scale = nn.Parameter(torch.full((3,), 0.01))

    def coefficients(self, X, z=None):
        """z: the stream mean of X when the caller has it already (bf16 [T, C])."""
        n = self.n
        if X.is_cuda and X.dtype == torch.bfloat16 and self.coef_proj.weight.shape[0] % 8 == 0:
            # stream mean without an fp32 copy of X, then the RMSNorm and GEMM kernels of this package
            from nanoplm_b200.ops import functional as ops
            zn = ops.norm(X.mean(dim=1) if z is None else z, self.coef_norm_weight, self.eps, rms=True)
            pre = ops.linear(zn, self.coef_proj.weight)
            if n in (2, 4) and 1 <= self.iters <= 8:
                return _CoefFn.apply(pre, self.static_alpha, self.static_beta, self.static_res, self.dyn_scale,
                                     max(1, self.iters), n)
            d = torch.tanh(pre.float())
        else:
            z = X.float().mean(dim=1)
            z = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + self.eps) * self.coef_norm_weight.float()
            d = torch.tanh(F.linear(z, self.coef_proj.weight.float()))
        s = self.dyn_scale.float()
        alpha = torch.softmax(self.static_alpha.float() + s[0] * d[:, :n], dim=-1)
        beta = 2.0 * torch.sigmoid(self.static_beta.float() + s[1] * d[:, n:2 * n])
        R = sinkhorn(self.static_res.float() + s[2] * d[:, 2 * n:].reshape(-1, n, n), self.iters)
        return alpha, beta, R

    def _threaded(self, X) -> bool:
        return (X.is_cuda and X.dtype == torch.bfloat16 and X.shape[-1] % 8 == 0 and X.shape[1] <= 4
                and self.coef_proj.weight.shape[0] % 8 == 0 and torch.is_grad_enabled() and X.requires_grad)

    def read(self, X):
        """Returns (h, state); `state` goes to `write` together with the same X."""
        if self._threaded(X):
            site = _SiteGrad()
            z, X1 = _MeanFn.apply(X.contiguous(), site)
            alpha, beta, R = self.coefficients(X1, z)
            h, X2 = _ReadThreadFn.apply(X1, alpha, site)
            return h, (beta, R, X2)
        alpha, beta, R = self.coefficients(X)
        return mhc_read(X, alpha), (beta, R, None)

    def write(self, X, y, state):
        beta, R, threaded = state
        return mhc_write(X if threaded is None else threaded, y, R, beta)
