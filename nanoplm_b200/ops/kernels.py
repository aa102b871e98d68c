"""Thin tensor-level wrappers over the C ABI of the sm_100a kernels (no autograd here).

Every function takes CUDA tensors, checks shapes / dtypes / contiguity, launches on the current
stream and returns output tensors. ``nanoplm_b200.ops.functional`` builds differentiable ops on top.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import _lib
from ._lib import check_rc, count_launch, lib, ptr, status_word, stream_ptr

EPI_STORE, EPI_ADD, EPI_ATOMIC_F32, EPI_GELU, EPI_STORE_F32, EPI_SWIGLU, EPI_ROPE, EPI_RELU = 0, 1, 2, 3, 4, 5, 6, 7
# acc = dL/dh of h = silu(gate) * value; aux = the [value | gate] pre-activations (2N wide);
# out = their gradient (2N wide)
EPI_SWIGLU_BWD = 8

_BF16 = torch.bfloat16


def _chk(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def _rowmajor(t: torch.Tensor, name: str) -> int:
    """Returns the row stride of a 2-D tensor whose last dim is contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dim")
    return t.stride(0)


# --------------------------------------------------------------------------- GEMM
import os as _os

_GEMM_PAIR_DEFAULT = [_os.environ.get("NPLM_GEMM_PAIR", "0") == "1"]


def set_gemm_pair_default(enabled: bool) -> None:
    """Default of gemm(pair=None): run qualifying GEMMs on CTA pairs (cta_group::2)."""
    _GEMM_PAIR_DEFAULT[0] = bool(enabled)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         epi: int = EPI_STORE, out: torch.Tensor | None = None, aux: torch.Tensor | None = None,
         splits: int = 1, bn: int | None = None, max_ctas: int = 0,
         direct_epilogue: bool = False, rope: tuple | None = None, pair: bool | None = None) -> torch.Tensor:
    """C[M,N] (+)= op(A) op(B)^T on tcgen05 tensor cores.

    a: [M,K] (a_mn=False) or [K,M] (a_mn=True); b: [N,K] (b_mn=False) or [K,N] (b_mn=True).
    epi: EPI_STORE / EPI_ADD (aux = residual) / EPI_ATOMIC_F32 (out fp32, accumulated in place) /
    EPI_GELU / EPI_RELU (aux = optional pre-activation output) / EPI_STORE_F32 / EPI_SWIGLU (out is N/2 wide,
    aux = optional [M,N] pre-activation output). bf16 outputs leave through shared memory and
    TMA stores; direct_epilogue=True selects per-thread global stores instead.
    EPI_ROPE: rope = (pos int32 [M], cos fp32 [P,32], sin fp32 [P,32], rope_cols): rotary embedding
    (head_dim 64) on every 64-wide head that starts below column rope_cols.
    pair: run on CTA pairs (tcgen05 cta_group::2, two SMs per 256 x 256 tile). None = the package
    default (`set_gemm_pair_default`); only 256-wide tiles without max_ctas qualify.
    """
    _chk(a, _BF16, "a")
    _chk(b, _BF16, "b")
    ag = getattr(b, "_ag", None)
    if ag is not None and ag.stale:
        # a row-sharded weight whose other row blocks are out of date (parameter-sharded data
        # parallelism): the first forward GEMM of the step gathers them from the peers inside the
        # kernel; any other consumer triggers an explicit gather
        if (not a_mn and not b_mn and splits == 1 and max_ctas == 0 and not direct_epilogue
                and epi in (EPI_STORE, EPI_ADD, EPI_GELU, EPI_RELU, EPI_SWIGLU, EPI_ROPE)):
            res = gemm_ag(a, b, ag.ptrs, ag.rank, ag.world, ag.flags, epi=epi, out=out, aux=aux, rope=rope)
            ag.stale = False
            return res
        ag.gather_now(b)
    lda, ldb = _rowmajor(a, "a"), _rowmajor(b, "b")
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"inner dims differ: {K} vs {Kb}")
    out_cols = N // 2 if epi == EPI_SWIGLU else (2 * N if epi == EPI_SWIGLU_BWD else N)
    f32_out = epi in (EPI_ATOMIC_F32, EPI_STORE_F32)
    if out is None:
        if epi == EPI_ATOMIC_F32:
            raise ValueError("EPI_ATOMIC_F32 needs an fp32 accumulator passed as out")
        out = torch.empty((M, out_cols), dtype=torch.float32 if f32_out else _BF16, device=a.device)
    _chk(out, torch.float32 if f32_out else _BF16, "out")
    if tuple(out.shape) != (M, out_cols):
        raise ValueError(f"out has shape {tuple(out.shape)}, expected {(M, out_cols)}")
    ldc = _rowmajor(out, "out")
    ldr = 0
    if aux is not None:
        _chk(aux, _BF16, "aux")
        ldr = _rowmajor(aux, "aux")
        aux_cols = 2 * N if epi == EPI_SWIGLU_BWD else N
        if tuple(aux.shape) != (M, aux_cols):
            raise ValueError(f"aux has shape {tuple(aux.shape)}, expected {(M, aux_cols)}")
    elif epi == EPI_ADD:
        raise ValueError("EPI_ADD needs the residual passed as aux")
    elif epi == EPI_SWIGLU_BWD:
        raise ValueError("EPI_SWIGLU_BWD needs the pre-activations passed as aux")
    if bn is None:
        bn = 256 if (N >= 256 or epi in (EPI_SWIGLU, EPI_SWIGLU_BWD)) else 128
    r_pos = r_cos = r_sin = None
    r_cols = 0
    if epi == EPI_ROPE:
        if rope is None:
            raise ValueError("EPI_ROPE needs rope=(pos, cos, sin, rope_cols)")
        r_pos, r_cos, r_sin, r_cols = rope
        _chk(r_pos, torch.int32, "rope pos")
        _chk(r_cos, torch.float32, "rope cos")
        if r_pos.numel() != M or r_cos.shape[-1] != 32:
            raise ValueError("rope tables must be [P, 32] and pos must have one entry per row")
    if pair is None:
        pair = _GEMM_PAIR_DEFAULT[0]
    if pair and bn == 256 and max_ctas == 0 and not (a_mn and not b_mn):
        rc = lib("gemm_tcgen05").nplm_gemm_bf16_pair(
            ptr(a), ptr(b), ptr(out), ptr(aux), c_int(M), c_int(N), c_int(K), c_int(lda), c_int(ldb),
            c_int(ldc), c_int(ldr), c_int(int(a_mn)), c_int(int(b_mn)), c_int(epi), c_int(splits),
            c_int(int(direct_epilogue)), ptr(r_pos), ptr(r_cos), ptr(r_sin),
            c_int(int(r_cols)), ptr(status_word(a.device)), stream_ptr())
        check_rc(rc, "gemm_bf16_pair")
        count_launch()
        return out
    rc = lib("gemm_tcgen05").nplm_gemm_bf16(
        ptr(a), ptr(b), ptr(out), ptr(aux), c_int(M), c_int(N), c_int(K), c_int(lda), c_int(ldb),
        c_int(ldc), c_int(ldr), c_int(int(a_mn)), c_int(int(b_mn)), c_int(epi), c_int(splits),
        c_int(bn), c_int(max_ctas), c_int(int(direct_epilogue)), ptr(r_pos), ptr(r_cos), ptr(r_sin),
        c_int(int(r_cols)), ptr(status_word(a.device)), stream_ptr())
    check_rc(rc, "gemm_bf16")
    count_launch()
    return out


def gemm_ag(a: torch.Tensor, b_full: torch.Tensor, b_ptrs, rank: int, world: int, flags: torch.Tensor, *,
            epi: int = EPI_STORE, out: torch.Tensor | None = None, aux: torch.Tensor | None = None,
            bn: int | None = None, rope: tuple | None = None) -> torch.Tensor:
    """All-gather fused into the GEMM: C = A B^T with B [N,K] row-sharded over `world` ranks.

    b_full is this rank's full-size weight buffer in peer-mapped (symmetric) memory, of which only
    rows [rank*N/world, (rank+1)*N/world) are valid on entry; b_ptrs is the ctypes array of all ranks'
    buffer addresses. The kernel pulls the other shards over NVLink while the tensor cores work on
    the local shard's tiles; afterwards b_full holds the whole matrix. flags: uint32/int32 [8].
    The caller orders the call after the peers' shard writes and before their next update.
    """
    _chk(a, _BF16, "a")
    _chk(b_full, _BF16, "b")
    M, K = a.shape
    N, Kb = b_full.shape
    if K != Kb:
        raise ValueError(f"inner dims differ: {K} vs {Kb}")
    if N % world:
        raise ValueError("rows of B must divide evenly over the ranks")
    rows = N // world
    unit = rows * 2 if epi == EPI_SWIGLU else rows     # a SwiGLU tile reads bn / 2 value rows and bn / 2 gate rows
    if bn is None:
        bn = 256 if unit % 256 == 0 else 128
    if unit % bn:
        raise ValueError(f"shard height {rows} does not hold whole {bn}-wide tiles")
    if epi == EPI_SWIGLU and (world % 2 or (N // 2) % rows):
        raise ValueError("SwiGLU with a row-sharded weight needs an even number of ranks")
    if out is None:
        out = torch.empty((M, N // 2 if epi == EPI_SWIGLU else N), dtype=_BF16, device=a.device)
    ldr = 0
    if aux is not None:
        ldr = _rowmajor(aux, "aux")
    r_pos, r_cos, r_sin, r_cols = rope if rope is not None else (None, None, None, 0)
    if epi == EPI_ROPE and rope is None:
        raise ValueError("EPI_ROPE needs rope=(pos, cos, sin, rope_cols)")
    rc = lib("gemm_tcgen05").nplm_gemm_bf16_ag_rope(
        ptr(a), b_ptrs, ptr(out), ptr(aux), c_int(M), c_int(N), c_int(K), c_int(_rowmajor(a, "a")),
        c_int(_rowmajor(b_full, "b")), c_int(_rowmajor(out, "out")), c_int(ldr), c_int(epi), c_int(bn),
        c_int(rank), c_int(world), ptr(flags), ptr(r_pos), ptr(r_cos), ptr(r_sin), c_int(r_cols),
        ptr(status_word(a.device)), stream_ptr())
    check_rc(rc, "gemm_bf16_ag")
    count_launch()
    return out


def wgrad_splits(n_out: int, k_in: int, tokens: int, bn: int = 256, sms: int = 148) -> int:
    """Split-K factor for a weight-gradient GEMM [n_out, k_in] reduced over `tokens`: the smallest
    factor (<= 4) whose work items fill the last wave of `sms` CTAs best."""
    tiles = ((n_out + 127) // 128) * ((k_in + bn - 1) // bn)
    kb = (tokens + 63) // 64
    best, best_eff = 1, 0.0
    for s in range(1, 5):
        if s > 1 and kb // s < 16:
            break
        work = tiles * s
        eff = work / (((work + sms - 1) // sms) * sms)
        if eff > best_eff + 0.02:
            best, best_eff = s, eff
    return best


# --------------------------------------------------------------------------- norms
def norm_fwd(x: torch.Tensor, w: torch.Tensor | None, eps: float, rms: bool = False,
             ids: torch.Tensor | None = None):
    """LayerNorm (no bias) / RMSNorm over the last dim. With ids, rows are table[ids] (embedding).

    Returns (y, mean, rstd); mean is None for RMSNorm.
    """
    _chk(x, _BF16, "x")
    C = x.shape[-1]
    if ids is not None:
        _chk(ids, torch.int32, "ids")
        T = ids.numel()
    else:
        T = x.numel() // C
    x2 = x.reshape(-1, C)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    y = torch.empty((T, C), dtype=_BF16, device=x.device)
    mean = None if rms else torch.empty(T, dtype=torch.float32, device=x.device)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    rc = lib("elementwise").nplm_norm_fwd(ptr(x2), ptr(ids), ptr(w), ptr(y), ptr(mean), ptr(rstd),
                                          c_int(T), c_int(C), c_float(eps), c_int(int(rms)),
                                          stream_ptr())
    check_rc(rc, "norm_fwd")
    count_launch()
    return y, mean, rstd


def norm_bwd(dy, x, w, mean, rstd, *, rms=False, dres=None, dw=None, ids=None, dtable=None):
    """Backward of norm_fwd. dw (fp32 [C]) and dtable (fp32 [V,C]) are accumulated in place.

    Returns dx (None in embedding mode)."""
    C = dy.shape[-1]
    T = dy.numel() // C
    dy2 = dy.reshape(T, C)
    if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
    dx = None if ids is not None else torch.empty((T, C), dtype=_BF16, device=dy.device)
    V = x.shape[0] if ids is not None else 0
    rc = lib("elementwise").nplm_norm_bwd(
        ptr(dy2), ptr(x), ptr(ids), ptr(w), ptr(mean), ptr(rstd), ptr(dres), ptr(dx), ptr(dw),
        ptr(dtable), c_int(T), c_int(C), c_int(V), c_int(int(rms)), stream_ptr())
    check_rc(rc, "norm_bwd")
    count_launch()
    return dx


# --------------------------------------------------------------------------- rope / swiglu / act
def rope_(qkv: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, H: int,
          D: int, backward: bool = False) -> torch.Tensor:
    """In-place rotary embedding on the q and k parts of qkv [T, 3*H*D]."""
    _chk(qkv, _BF16, "qkv")
    _chk(pos, torch.int32, "pos")
    T = qkv.shape[0]
    rc = lib("elementwise").nplm_rope(ptr(qkv), ptr(pos), ptr(cos), ptr(sin), c_int(T), c_int(H),
                                      c_int(D), c_int(int(backward)), stream_ptr())
    check_rc(rc, "rope")
    count_launch()
    return qkv


def swiglu_fwd(pre: torch.Tensor) -> torch.Tensor:
    T, two_i = pre.shape
    out = torch.empty((T, two_i // 2), dtype=_BF16, device=pre.device)
    rc = lib("elementwise").nplm_swiglu_fwd(ptr(pre), ptr(out), c_longlong(T), c_int(two_i // 2),
                                            stream_ptr())
    check_rc(rc, "swiglu_fwd")
    count_launch()
    return out


def swiglu_bwd(pre: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    T, two_i = pre.shape
    dpre = torch.empty_like(pre)
    rc = lib("elementwise").nplm_swiglu_bwd(ptr(pre), ptr(dout), ptr(dpre), c_longlong(T),
                                            c_int(two_i // 2), stream_ptr())
    check_rc(rc, "swiglu_bwd")
    count_launch()
    return dpre


_ACT = {"gelu": 0, "relu": 1, "silu": 2}


def act_fwd(pre: torch.Tensor, act: str) -> torch.Tensor:
    out = torch.empty_like(pre)
    rc = lib("elementwise").nplm_act_fwd(ptr(pre), ptr(out), c_longlong(pre.numel()),
                                         c_int(_ACT[act]), stream_ptr())
    check_rc(rc, "act_fwd")
    count_launch()
    return out


def act_bwd(pre: torch.Tensor, dout: torch.Tensor, act: str) -> torch.Tensor:
    dpre = torch.empty_like(pre)
    rc = lib("elementwise").nplm_act_bwd(ptr(pre), ptr(dout), ptr(dpre), c_longlong(pre.numel()),
                                         c_int(_ACT[act]), stream_ptr())
    check_rc(rc, "act_bwd")
    count_launch()
    return dpre


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    n, C = idx.numel(), src.shape[1]
    dst = torch.empty((n, C), dtype=_BF16, device=src.device)
    rc = lib("elementwise").nplm_gather_rows(ptr(src), ptr(idx), ptr(dst), c_int(n), c_int(C),
                                             stream_ptr())
    check_rc(rc, "gather_rows")
    count_launch()
    return dst


def scatter_rows_(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    n, C = idx.numel(), src.shape[1]
    rc = lib("elementwise").nplm_scatter_rows(ptr(src), ptr(idx), ptr(dst), c_int(n), c_int(C),
                                              stream_ptr())
    check_rc(rc, "scatter_rows")
    count_launch()
    return dst


# --------------------------------------------------------------------------- cross entropy
def ce_fwd(h, W, bias, labels, inv_count, want_logits=False):
    n, C = h.shape
    V = W.shape[0]
    dlogits = torch.empty((n, 32), dtype=torch.float32, device=h.device)
    logits = torch.empty((n, V), dtype=torch.float32, device=h.device) if want_logits else None
    loss = torch.zeros(1, dtype=torch.float32, device=h.device)
    rc = lib("elementwise").nplm_ce_fwd(ptr(h), ptr(W), ptr(bias), ptr(labels), ptr(inv_count),
                                        ptr(dlogits), ptr(logits), ptr(loss), c_int(n), c_int(C),
                                        c_int(V), stream_ptr())
    check_rc(rc, "ce_fwd")
    count_launch()
    return loss, dlogits, logits


def ce_bwd(h, W, dlogits, gscale, dW, dbias):
    n, C = h.shape
    V = W.shape[0]
    dh = torch.empty_like(h)
    rc = lib("elementwise").nplm_ce_bwd(ptr(h), ptr(W), ptr(dlogits), ptr(gscale), ptr(dh), ptr(dW),
                                        ptr(dbias), c_int(n), c_int(C), c_int(V), stream_ptr())
    check_rc(rc, "ce_bwd")
    count_launch()
    return dh


# --------------------------------------------------------------------------- optimizer
def sumsq_(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    rc = lib("elementwise").nplm_sumsq(ptr(x), c_longlong(x.numel()), ptr(out), stream_ptr())
    check_rc(rc, "sumsq")
    count_launch()
    return out


def adamw_(p, m, v, g, p_bf16, hyper, sumsq, zero_grad=True) -> None:
    rc = lib("elementwise").nplm_adamw(ptr(p), ptr(m), ptr(v), ptr(g), ptr(p_bf16), ptr(hyper),
                                       ptr(sumsq), c_longlong(p.numel()), c_int(int(zero_grad)),
                                       stream_ptr())
    check_rc(rc, "adamw")
    count_launch()


def muon_momentum_(g, m, offsets, numel: int, upd, usq, sumsq, grad_scale: float, max_norm: float,
                   mu: float, nesterov: bool) -> None:
    """Momentum update of the matrices at flat `offsets` (int64, device) of g / m (fp32 flat
    buffers); writes the bf16 Newton-Schulz input `upd` [n, numel] and adds its squared Frobenius
    norms to `usq` [n]."""
    rc = lib("elementwise").nplm_muon_momentum(
        ptr(g), ptr(m), ptr(offsets), c_int(offsets.numel()), c_longlong(numel), ptr(upd), ptr(usq),
        ptr(sumsq), c_float(grad_scale), c_float(max_norm), c_float(mu), c_int(int(nesterov)), stream_ptr())
    check_rc(rc, "muon_momentum")
    count_launch()


def muon_apply_(p, p_bf16, offsets, numel: int, O, lr: float, wd: float, cautious: bool) -> None:
    """p[offsets[i] : +numel] -= lr * (wd-term + O[i]) for the bf16 stack O [n, numel]; also
    writes the bf16 copy of the parameters."""
    rc = lib("elementwise").nplm_muon_apply(
        ptr(p), ptr(p_bf16), ptr(offsets), c_int(offsets.numel()), c_longlong(numel), ptr(O),
        c_float(lr), c_float(wd), c_int(int(cautious)), stream_ptr())
    check_rc(rc, "muon_apply")
    count_launch()


def adamw_slots_(p, m, v, g, p_bf16, offsets, numels, decay, max_numel: int, sumsq, grad_scale: float,
                 max_norm: float, lr: float, beta1: float, beta2: float, eps: float, wd: float,
                 bc1: float, bc2: float) -> None:
    """AdamW on the tensors listed in (offsets, numels, decay) of one flat buffer, one launch."""
    rc = lib("elementwise").nplm_adamw_slots(
        ptr(p), ptr(m), ptr(v), ptr(g), ptr(p_bf16), ptr(offsets), ptr(numels), ptr(decay),
        c_int(offsets.numel()), c_longlong(max_numel), ptr(sumsq), c_float(grad_scale), c_float(max_norm),
        c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(wd), c_float(bc1), c_float(bc2),
        stream_ptr())
    check_rc(rc, "adamw_slots")
    count_launch()


def cast_f32_bf16_(src: torch.Tensor, dst: torch.Tensor) -> None:
    rc = lib("elementwise").nplm_cast_f32_bf16(ptr(src), ptr(dst), c_longlong(src.numel()),
                                               stream_ptr())
    check_rc(rc, "cast")
    count_launch()


def masked_mse(s, t, valid, inv_count, want_grad=True):
    T, C = s.shape
    ds = torch.empty_like(s) if want_grad else None
    loss = torch.zeros(1, dtype=torch.float32, device=s.device)
    rc = lib("elementwise").nplm_masked_mse(ptr(s), ptr(t), ptr(valid), ptr(inv_count), ptr(ds),
                                            ptr(loss), c_int(T), c_int(C), stream_ptr())
    check_rc(rc, "masked_mse")
    count_launch()
    return loss, ds


# --------------------------------------------------------------------------- attention
def seq_bounds(cu_seqlens: torch.Tensor, T: int):
    _chk(cu_seqlens, torch.int32, "cu_seqlens")
    s = torch.empty(T, dtype=torch.int32, device=cu_seqlens.device)
    e = torch.empty(T, dtype=torch.int32, device=cu_seqlens.device)
    rc = lib("attention").nplm_seq_bounds(ptr(cu_seqlens), c_int(cu_seqlens.numel() - 1), ptr(s),
                                          ptr(e), c_int(T), stream_ptr())
    check_rc(rc, "seq_bounds")
    count_launch()
    return s, e


_FA_IMPL = [_os.environ.get("NPLM_FA_IMPL", "ws")]


def set_attention_impl(name: str) -> None:
    """"ws": the persistent warp-specialised kernels (attention_ws.cu, default);
    "single": the one-role-per-CTA kernels of attention.cu."""
    if name not in ("ws", "single"):
        raise ValueError("attention impl must be 'ws' or 'single'")
    _FA_IMPL[0] = name


def fa_fwd(qkv, seq_start, seq_end, H, D, window, scale, impl: str | None = None, max_ctas: int = 0):
    _chk(qkv, _BF16, "qkv")
    T = qkv.shape[0]
    out = torch.empty((T, H * D), dtype=_BF16, device=qkv.device)
    lse = torch.empty((H, T), dtype=torch.float32, device=qkv.device)
    if (impl or _FA_IMPL[0]) == "ws":
        rc = lib("attention_ws").nplm_fa_fwd_ws(ptr(qkv), ptr(out), ptr(lse), ptr(seq_start), ptr(seq_end),
                                                c_int(T), c_int(H), c_int(D), c_int(window), c_float(scale),
                                                c_int(max_ctas), ptr(status_word(qkv.device)), stream_ptr())
    else:
        rc = lib("attention").nplm_fa_fwd(ptr(qkv), ptr(out), ptr(lse), ptr(seq_start), ptr(seq_end),
                                          c_int(T), c_int(H), c_int(D), c_int(window), c_float(scale),
                                          ptr(status_word(qkv.device)), stream_ptr())
    check_rc(rc, "fa_fwd")
    count_launch()
    return out, lse


def gemm_dgrad_delta(dy: torch.Tensor, w: torch.Tensor, o: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """dO = dy @ w (w [K, N] read MN-major) in bf16 and, from the same epilogue,
    delta[h, t] = sum over head h's 64 columns of dO[t] * o[t] (fp32 [N / 64, T])."""
    _chk(dy, _BF16, "dy")
    _chk(w, _BF16, "w")
    _chk(o, _BF16, "o")
    _chk(delta, torch.float32, "delta")
    M, Kd = dy.shape
    if w.shape[0] != Kd:
        raise ValueError("inner dims differ")
    N = w.shape[1]
    if N % 64 or tuple(o.shape) != (M, N) or tuple(delta.shape) != (N // 64, M) or not delta.is_contiguous():
        raise ValueError("o must be [M, N], delta [N / 64, M] contiguous, N a multiple of 64")
    out = torch.empty((M, N), dtype=_BF16, device=dy.device)
    rc = lib("gemm_tcgen05").nplm_gemm_bf16_delta(
        ptr(dy), ptr(w), ptr(out), ptr(o), ptr(delta), c_int(M), c_int(N), c_int(Kd), c_int(_rowmajor(dy, "dy")),
        c_int(_rowmajor(w, "w")), c_int(N), c_int(_rowmajor(o, "o")), c_int(1), ptr(status_word(dy.device)),
        stream_ptr())
    check_rc(rc, "gemm_bf16_delta")
    count_launch()
    return out


_FA_DETERMINISTIC = [_os.environ.get("NPLM_FA_DETERMINISTIC", "0") not in ("", "0")]


def set_attention_deterministic(flag: bool) -> None:
    """True: the warp-specialised backward pass forms dQ in a second, query-stationary launch instead
    of fp32 atomics, so two runs on the same inputs give the same bits (about 1.4x the time)."""
    _FA_DETERMINISTIC[0] = bool(flag)


def fa_bwd(qkv, out, dout, lse, seq_start, seq_end, H, D, window, scale, dq_acc=None, delta=None,
           rope: tuple | None = None, delta_ready: bool = False, impl: str | None = None, max_ctas: int = 0,
           deterministic: bool | None = None):
    """rope = (pos, cos, sin): q / k in qkv were rotated before the forward pass; dQ / dK are rotated
    back inside the kernels. delta_ready: `delta` [H, T] already holds rowsum(dO * O) (see
    gemm_dgrad_delta); the kernel that computes it from out and dout is skipped. deterministic (default:
    `set_attention_deterministic`): no atomics, bitwise reproducible (warp-specialised kernels only)."""
    T = qkv.shape[0]
    dqkv = torch.empty_like(qkv)
    use_ws = (impl or _FA_IMPL[0]) == "ws"
    det = use_ws and (_FA_DETERMINISTIC[0] if deterministic is None else deterministic)
    if dq_acc is None and not det:
        dq_acc = torch.empty((T, H * D), dtype=torch.float32, device=qkv.device)
    if delta is None:
        delta = torch.empty((H, T), dtype=torch.float32, device=qkv.device)
    if not dout.is_contiguous():
        dout = dout.contiguous()
    r_pos, r_cos, r_sin = rope if rope is not None else (None, None, None)
    if delta_ready:
        out = None
    if use_ws:
        rc = lib("attention_ws").nplm_fa_bwd_ws_mode(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv),
                                                     ptr(dq_acc), ptr(delta), ptr(seq_start), ptr(seq_end),
                                                     c_int(T), c_int(H), c_int(D), c_int(window), c_float(scale),
                                                     ptr(r_pos), ptr(r_cos), ptr(r_sin), c_int(max_ctas),
                                                     c_int(3 if det else -1),
                                                     ptr(status_word(qkv.device)), stream_ptr())
    else:
        rc = lib("attention").nplm_fa_bwd_rope(ptr(qkv), ptr(out), ptr(dout), ptr(lse), ptr(dqkv),
                                               ptr(dq_acc), ptr(delta), ptr(seq_start), ptr(seq_end),
                                               c_int(T), c_int(H), c_int(D), c_int(window), c_float(scale),
                                               ptr(r_pos), ptr(r_cos), ptr(r_sin),
                                               ptr(status_word(qkv.device)), stream_ptr())
    check_rc(rc, "fa_bwd")
    count_launch(3 if delta_ready else 4)
    return dqkv


def fa_bias_fwd(qkv: torch.Tensor, seq_start: torch.Tensor, seq_end: torch.Tensor, bias: torch.Tensor,
                H: int, D: int, scale: float = 1.0) -> torch.Tensor:
    """Inference attention with a relative-position bias (T5-style teacher).

    qkv bf16 [T, 3*H*D] (q | k | v, head-major), seq_start / seq_end int32 [T] (key range of every
    token), bias fp32 [H, 2*S-1] indexed by key - query + S - 1. Returns bf16 [T, H*D]."""
    _chk(qkv, _BF16, "qkv")
    _chk(seq_start, torch.int32, "seq_start")
    _chk(seq_end, torch.int32, "seq_end")
    _chk(bias, torch.float32, "bias")
    T = qkv.shape[0]
    S = (bias.shape[1] + 1) // 2
    out = torch.empty((T, H * D), dtype=_BF16, device=qkv.device)
    rc = lib("attention_bias").nplm_fa_bias_fwd(ptr(qkv), ptr(out), ptr(seq_start), ptr(seq_end),
                                                ptr(bias.contiguous()), c_int(T), c_int(H), c_int(D), c_int(S),
                                                c_float(scale), ptr(status_word(qkv.device)), stream_ptr())
    check_rc(rc, "fa_bias_fwd")
    count_launch()
    return out


def check_status() -> None:
    _lib.check_status()


# --------------------------------------------------------------------------- conv / mHC
def dwconv(x, w, bias, seq_start, seq_end, flip=False):
    T, C = x.shape
    KS = w.shape[1]
    y = torch.empty_like(x)
    rc = lib("extras").nplm_dwconv(ptr(x), ptr(w), ptr(bias), ptr(seq_start), ptr(seq_end), ptr(y), c_int(T),
                                   c_int(C), c_int(KS), c_int(int(flip)), stream_ptr())
    check_rc(rc, "dwconv")
    count_launch()
    return y


def dwconv_bwd_w(x, dy, seq_start, seq_end, dw, dbias):
    T, C = x.shape
    KS = dw.shape[1]
    rc = lib("extras").nplm_dwconv_bwd_w(ptr(x), ptr(dy), ptr(seq_start), ptr(seq_end), ptr(dw), ptr(dbias),
                                         c_int(T), c_int(C), c_int(KS), stream_ptr())
    check_rc(rc, "dwconv_bwd_w")
    count_launch()


def mhc_read(X, alpha):
    T, n, C = X.shape
    h = torch.empty((T, C), dtype=_BF16, device=X.device)
    rc = lib("extras").nplm_mhc_read(ptr(X), ptr(alpha), ptr(h), c_int(T), c_int(n), c_int(C), stream_ptr())
    check_rc(rc, "mhc_read")
    count_launch()
    return h


def mhc_write(X, y, R, beta):
    T, n, C = X.shape
    Xn = torch.empty_like(X)
    rc = lib("extras").nplm_mhc_write(ptr(X), ptr(y), ptr(R), ptr(beta), ptr(Xn), c_int(T), c_int(n), c_int(C),
                                      stream_ptr())
    check_rc(rc, "mhc_write")
    count_launch()
    return Xn


def mhc_mean(X):
    """Mean over the streams: X [T, n, C] bf16 -> [T, C]."""
    T, n, C = X.shape
    z = torch.empty((T, C), dtype=_BF16, device=X.device)
    rc = lib("extras").nplm_mhc_mean(ptr(X), ptr(z), c_int(T), c_int(n), c_int(C), stream_ptr())
    check_rc(rc, "mhc_mean")
    count_launch()
    return z


def mhc_dx_combine(g, alpha, dh, dz, shape):
    """dX = g + alpha[:, :, None] * dh[:, None, :] + dz[:, None, :] / n in one pass (any of the three
    terms may be None); shape = (T, n, C)."""
    T, n, C = shape
    ref = next(t for t in (g, dh, dz) if t is not None)
    dX = torch.empty((T, n, C), dtype=_BF16, device=ref.device)
    rc = lib("extras").nplm_mhc_dx_combine(ptr(g), ptr(alpha), ptr(dh), ptr(dz), ptr(dX), c_int(T), c_int(n),
                                           c_int(C), stream_ptr())
    check_rc(rc, "mhc_dx_combine")
    count_launch()
    return dX


def mhc_bwd(X, y, R, alpha, beta, dXn, dh, want_dx: bool = True):
    """Backward of write (dXn given) and / or read (dh given). Returns (dX, dy, dR, dalpha, dbeta);
    want_dx=False skips the dX output (only the coefficient gradients are computed)."""
    T, n, C = X.shape
    dev = X.device
    dX = torch.empty_like(X) if want_dx else None
    dy = torch.empty((T, C), dtype=_BF16, device=dev) if dXn is not None else None
    dR = torch.empty((T, n, n), dtype=torch.float32, device=dev) if dXn is not None else None
    dbeta = torch.empty((T, n), dtype=torch.float32, device=dev) if dXn is not None else None
    dalpha = torch.empty((T, n), dtype=torch.float32, device=dev) if dh is not None else None
    rc = lib("extras").nplm_mhc_bwd(ptr(X), ptr(y), ptr(R), ptr(alpha), ptr(beta), ptr(dXn), ptr(dh), ptr(dX),
                                    ptr(dy), ptr(dR), ptr(dalpha), ptr(dbeta), c_int(T), c_int(n), c_int(C),
                                    stream_ptr())
    check_rc(rc, "mhc_bwd")
    count_launch()
    return dX, dy, dR, dalpha, dbeta


# --------------------------------------------------------------------------- device-side MLM masking
def mhc_coef_fwd(pre, a, b, r, s, iters: int, n: int):
    """Raw coefficient projections pre bf16 [T, 2n+n*n] -> (alpha [T,n], beta [T,n], R [T,n,n]) fp32.
    a, b [n], r [n,n], s [3]: fp32 static parts and dynamic scales."""
    _chk(pre, _BF16, "pre")
    T = pre.shape[0]
    dev = pre.device
    alpha = torch.empty((T, n), dtype=torch.float32, device=dev)
    beta = torch.empty((T, n), dtype=torch.float32, device=dev)
    R = torch.empty((T, n, n), dtype=torch.float32, device=dev)
    rc = lib("extras").nplm_mhc_coef_fwd(ptr(pre), ptr(a), ptr(b), ptr(r), ptr(s), c_int(iters), c_int(T),
                                         c_int(n), ptr(alpha), ptr(beta), ptr(R), stream_ptr())
    check_rc(rc, "mhc_coef_fwd")
    count_launch()
    return alpha, beta, R


def mhc_coef_bwd(pre, a, b, r, s, iters: int, n: int, dalpha, dbeta, dR, da, db, dr, ds):
    """Backward of mhc_coef_fwd. Returns dpre (bf16); da, db, dr, ds (fp32) are accumulated in place."""
    T = pre.shape[0]
    dpre = torch.empty_like(pre)
    rc = lib("extras").nplm_mhc_coef_bwd(ptr(pre), ptr(a), ptr(b), ptr(r), ptr(s), c_int(iters), c_int(T),
                                         c_int(n), ptr(dalpha), ptr(dbeta), ptr(dR), ptr(dpre), ptr(da), ptr(db),
                                         ptr(dr), ptr(ds), stream_ptr())
    check_rc(rc, "mhc_coef_bwd")
    count_launch()
    return dpre


def mlm_mask(ids: torch.Tensor, n_real: int, special_ids, mask_id: int, pool: torch.Tensor, p_sel: float,
             p_mask: float, p_rand: float, seed: int, step: int):
    """Philox masking of flat int64 ids on the device. Returns (corrupted ids, labels)."""
    from ctypes import c_ulonglong
    _chk(ids, torch.int64, "ids")
    _chk(pool, torch.int32, "pool")
    bits = 0
    for s in special_ids:
        bits |= 1 << int(s)
    out, labels = torch.empty_like(ids), torch.empty_like(ids)
    rc = lib("extras").nplm_mlm_mask(ptr(ids), ptr(out), ptr(labels), c_int(ids.numel()), c_int(int(n_real)),
                                     c_ulonglong(bits), c_int(mask_id), ptr(pool), c_int(pool.numel()),
                                     c_float(p_sel), c_float(p_mask), c_float(p_rand), c_ulonglong(seed),
                                     c_ulonglong(step), stream_ptr())
    check_rc(rc, "mlm_mask")
    count_launch()
    return out, labels
