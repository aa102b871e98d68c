"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _k():
    from nanoplm_b200.ops import kernels
    return kernels


def _randn(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(BF)


def _close(a, b, rtol=2e-2, atol=2e-2, what=""):
    a = a.float()
    b = b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, rtol=rtol, atol=atol * max(1.0, ref)), f"{what}: max err {err} (ref max {ref})"


def _close_gemm(c, ref, K, scale=1.0, what=""):
    """Per-element bound for a bf16 result of a K-long fp32-accumulated contraction of bf16 inputs:
    |c - ref| <= 2^-7 |ref| + 0.25 sqrt(K) 2^-8 scale (scale = product of the operands' standard
    deviations). The first term covers the bf16 rounding of the result with a factor 2 to spare, the
    second keeps elements near zero from failing on the rounding of their neighbours' magnitude; a
    dropped or doubled k-block changes an element by about sqrt(64) scale and is caught."""
    c, ref = c.float(), ref.float()
    bound = 2.0 ** -7 * ref.abs() + 0.25 * math.sqrt(K) * 2.0 ** -8 * scale
    bad = (c - ref).abs() > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} elements outside the per-element bound, worst excess "
                           f"{((c - ref).abs() - bound).max().item():.4g}")


# ------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (384, 512, 320), (300, 264, 200),
                                   (1000, 1024, 1024), (4096, 3072, 1024), (1, 128, 64), (7, 256, 128),
                                   (129, 128, 192), (4097, 256, 64)])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("direct", [False, True])
def test_gemm_kk(M, N, K, bn, direct, cuda_status):
    k = _k()
    a, b = _randn(M, K), _randn(N, K)
    c = k.gemm(a, b, bn=bn, direct_epilogue=direct)
    ref = a.float() @ b.float().t()
    _close_gemm(c, ref, K, what=f"gemm {M}x{N}x{K} bn{bn} direct={direct}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 320, 200), (1024, 1024, 4096)])
def test_gemm_majors(a_mn, b_mn, M, N, K, cuda_status):
    k = _k()
    a = _randn(K, M) if a_mn else _randn(M, K)
    b = _randn(K, N) if b_mn else _randn(N, K)
    for bn in (128, 256):
        c = k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
        af = a.float().t() if a_mn else a.float()
        bf = b.float() if b_mn else b.float().t()
        _close_gemm(c, af @ bf, K, what=f"gemm majors a_mn={a_mn} b_mn={b_mn} {M}x{N}x{K} bn{bn}")


@pytest.mark.parametrize("direct", [False, True])
@pytest.mark.parametrize("M,N,K", [(512, 768, 256), (1000, 1200, 192), (77, 144, 64)])
def test_gemm_epilogues(direct, M, N, K, cuda_status):
    k = _k()
    a, b = _randn(M, K), _randn(N, K, scale=0.1)
    ref = a.float() @ b.float().t()
    res = _randn(M, N)
    for bn in (128, 256):
        _close_gemm(k.gemm(a, b, epi=k.EPI_ADD, aux=res, bn=bn, direct_epilogue=direct), ref + res.float(),
                    K, scale=0.1, what=f"epi add bn{bn}")
        pre = torch.zeros(M, N, dtype=BF, device="cuda")
        out = k.gemm(a, b, epi=k.EPI_GELU, aux=pre, bn=bn, direct_epilogue=direct)
        _close_gemm(pre, ref, K, scale=0.1, what="gelu pre")
        _close(out, F.gelu(pre.float()), what="gelu out")
        # swiglu: b = [value rows | gate rows]
        pre2 = torch.zeros(M, N, dtype=BF, device="cuda")
        out2 = k.gemm(a, b, epi=k.EPI_SWIGLU, aux=pre2, bn=bn, direct_epilogue=direct)
        _close_gemm(pre2, ref, K, scale=0.1, what=f"swiglu pre bn{bn}")
        v, g = pre2.float().chunk(2, dim=-1)
        _close(out2, F.silu(g) * v, what=f"swiglu out bn{bn}")
        assert out2.shape == (M, N // 2)
    _close(k.gemm(a, b, epi=k.EPI_STORE_F32), ref, what="epi f32")


def test_gemm_output_canaries(cuda_status):
    """The staged epilogue must not write outside [M, N] of a larger allocation."""
    k = _k()
    M, N, K = 200, 136, 128
    a, b = _randn(M, K), _randn(N, K)
    big = torch.full((M + 64, N + 120), 7.0, dtype=BF, device="cuda")
    out = big[:M, :N]
    k.gemm(a, b, out=out)
    _close_gemm(out, a.float() @ b.float().t(), K, what="canary result")
    assert (big[M:, :] == 7).all() and (big[:, N:] == 7).all()


@pytest.mark.parametrize("splits", [1, 3, 8])
def test_gemm_wgrad_atomic(splits, cuda_status):
    k = _k()
    T, N, K = 2048, 256, 384          # dW[N,K] = dY[T,N]^T X[T,K]
    dy, x = _randn(T, N, scale=0.1), _randn(T, K)
    acc = torch.ones(N, K, dtype=torch.float32, device="cuda")
    k.gemm(dy, x, a_mn=True, b_mn=True, epi=k.EPI_ATOMIC_F32, out=acc, splits=splits)
    ref = 1.0 + dy.float().t() @ x.float()
    _close(acc, ref, what=f"wgrad splits={splits}")


def test_gemm_strided_views(cuda_status):
    """Operands that are column slices of a wider buffer (row stride > width)."""
    k = _k()
    big = _randn(512, 1024)
    a = big[:, 128:384]                 # [512, 256], row stride 1024
    b = _randn(192, 256)
    out_big = torch.zeros(512, 512, dtype=BF, device="cuda")
    out = out_big[:, 64:256]
    k.gemm(a, b, out=out)
    _close_gemm(out, a.float() @ b.float().t(), 256, what="strided")
    assert out_big[:, :64].abs().max().item() == 0 and out_big[:, 256:].abs().max().item() == 0


# ------------------------------------------------------------------------------- norms
@pytest.mark.parametrize("C,T", [(128, 777), (768, 777), (1024, 777), (1024, 1), (1024, 7), (256, 129),
                                 (128, 4097)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(C, T, rms, cuda_status):
    k = _k()
    x = _randn(T, C)
    w = (1 + 0.1 * torch.randn(C, device="cuda")).to(BF)
    dy = _randn(T, C)
    dres = _randn(T, C)
    y, mean, rstd = k.norm_fwd(x, w, 1e-5, rms=rms)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    if rms:
        ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    else:
        ref = F.layer_norm(xf, (C,), wf, None, 1e-5)
    _close(y, ref, what="norm fwd")
    ref.backward(dy.float())
    dw = torch.zeros(C, dtype=torch.float32, device="cuda")
    dx = k.norm_bwd(dy, x, w, mean, rstd, rms=rms, dres=dres, dw=dw)
    _close(dx, xf.grad + dres.float(), what="norm dx")
    _close(dw, wf.grad, rtol=3e-2, atol=3e-2, what="norm dw")


def test_embed_norm(cuda_status):
    k = _k()
    V, C, T = 32, 1024, 3000
    table = _randn(V, C, scale=0.02)
    w = (1 + 0.1 * torch.randn(C, device="cuda")).to(BF)
    ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    y, mean, rstd = k.norm_fwd(table, w, 1e-5, ids=ids)
    tf = table.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    ref = F.layer_norm(F.embedding(ids.long(), tf), (C,), wf, None, 1e-5)
    _close(y, ref, what="embed fwd")
    dy = _randn(T, C)
    ref.backward(dy.float())
    dtable = torch.zeros(V, C, dtype=torch.float32, device="cuda")
    dw = torch.zeros(C, dtype=torch.float32, device="cuda")
    k.norm_bwd(dy, table, w, mean, rstd, ids=ids, dtable=dtable, dw=dw)
    _close(dtable, tf.grad, rtol=3e-2, atol=3e-2, what="embed dtable")
    _close(dw, wf.grad, rtol=3e-2, atol=3e-2, what="embed dw")


# ------------------------------------------------------------------------------- rope / swiglu / act
def _rope_ref(x, cos, sin):
    x1, x2 = x.chunk(2, dim=-1)
    rot = torch.cat((-x2, x1), dim=-1)
    return x * cos + rot * sin


def test_rope(cuda_status):
    k = _k()
    T, H, D = 1000, 4, 64
    qkv = _randn(T, 3 * H * D)
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(512, device="cuda").float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    ref = qkv.float().view(T, 3, H, D).clone()
    c = torch.cat((cos, cos), -1)[pos.long()][:, None, :]
    s = torch.cat((sin, sin), -1)[pos.long()][:, None, :]
    ref[:, 0] = _rope_ref(ref[:, 0], c, s)
    ref[:, 1] = _rope_ref(ref[:, 1], c, s)
    orig = qkv.clone()
    k.rope_(qkv, pos, cos, sin, H, D)
    _close(qkv.view(T, 3, H, D), ref, what="rope fwd")
    # backward of a rotation is the inverse rotation
    k.rope_(qkv, pos, cos, sin, H, D, backward=True)
    _close(qkv, orig, what="rope bwd")


def test_swiglu_and_act(cuda_status):
    k = _k()
    T, I = 500, 256
    pre = _randn(T, 2 * I)
    dout = _randn(T, I)
    pf = pre.float().requires_grad_(True)
    v, g = pf.chunk(2, -1)
    ref = F.silu(g) * v
    _close(k.swiglu_fwd(pre), ref, what="swiglu fwd")
    ref.backward(dout.float())
    _close(k.swiglu_bwd(pre, dout), pf.grad, what="swiglu bwd")
    for name, fn in (("gelu", F.gelu), ("relu", F.relu), ("silu", F.silu)):
        p = _randn(T, I)
        pf = p.float().requires_grad_(True)
        r = fn(pf)
        _close(k.act_fwd(p, name), r, what=f"{name} fwd")
        r.backward(dout.float())
        _close(k.act_bwd(p, dout, name), pf.grad, what=f"{name} bwd")


def test_gather_scatter(cuda_status):
    k = _k()
    src = _randn(1000, 256)
    idx = torch.randperm(1000, device="cuda")[:300].to(torch.int32)
    g = k.gather_rows(src, idx)
    assert torch.equal(g, src[idx.long()])
    dst = torch.zeros(1000, 256, dtype=BF, device="cuda")
    k.scatter_rows_(dst, idx, g)
    ref = torch.zeros_like(dst)
    ref[idx.long()] = g
    assert torch.equal(dst, ref)


# ------------------------------------------------------------------------------- cross entropy
@pytest.mark.parametrize("V,C", [(32, 1024), (28, 1024), (32, 128), (32, 768)])
def test_cross_entropy(V, C, cuda_status):
    k = _k()
    n = 3001
    h = _randn(n, C)
    W = _randn(V, C, scale=0.05)
    bias = _randn(V, scale=0.1)
    labels = torch.randint(0, V, (n,), device="cuda", dtype=torch.int32)
    labels[::7] = -100
    nvalid = (labels >= 0).sum().float()
    inv = (1.0 / nvalid).reshape(1)
    loss, dlogits, logits = k.ce_fwd(h, W, bias, labels, inv, want_logits=True)
    hf, Wf, bf = h.float().requires_grad_(True), W.float().requires_grad_(True), bias.float().requires_grad_(True)
    ref_logits = hf @ Wf.t() + bf
    ref = F.cross_entropy(ref_logits, labels.long(), ignore_index=-100)
    _close(logits, ref_logits, what="ce logits")
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1, abs(ref.item())), (loss.item(), ref.item())
    (ref * 0.5).backward()
    gs = torch.full((1,), 0.5, device="cuda")
    dW = torch.zeros(V, C, dtype=torch.float32, device="cuda")
    db = torch.zeros(V, dtype=torch.float32, device="cuda")
    dh = k.ce_bwd(h, W, dlogits, gs, dW, db)
    _close(dh, hf.grad, rtol=3e-2, atol=3e-2, what="ce dh")
    _close(dW, Wf.grad, rtol=3e-2, atol=3e-2, what="ce dW")
    _close(db, bf.grad, rtol=3e-2, atol=3e-2, what="ce dbias")


# ------------------------------------------------------------------------------- optimizer
def test_adamw_and_sumsq(cuda_status):
    k = _k()
    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 3
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    pb = torch.empty(n, dtype=BF, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    ss = torch.zeros(1, device="cuda")
    k.sumsq_(g, ss)
    assert abs(ss.item() - g.double().pow(2).sum().item()) / ss.item() < 1e-4
    for step in range(1, 4):
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        hyper = torch.tensor([1e-2, 0.9, 0.999, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.999 ** step, 1.0, 1.0],
                             device="cuda")
        gg = g.clone()
        k.adamw_(p, m, v, gg, pb, hyper, ss, zero_grad=True)
        assert gg.abs().max().item() == 0
    _close(p, ref_p.detach(), rtol=1e-4, atol=1e-5, what="adamw p")
    _close(pb, ref_p.detach(), what="adamw bf16 copy")


def test_masked_mse(cuda_status):
    k = _k()
    T, C = 999, 1024
    s, t = _randn(T, C), _randn(T, C)
    valid = (torch.rand(T, device="cuda") > 0.3).to(torch.int32)
    inv = (1.0 / valid.sum().clamp(min=1).float()).reshape(1)
    loss, ds = k.masked_mse(s, t, valid, inv)
    sf = s.float().requires_grad_(True)
    ref = (((sf - t.float()) ** 2) * valid[:, None].float()).sum() / valid.sum().clamp(min=1)
    ref.backward()
    assert abs(loss.item() - ref.item()) / ref.item() < 1e-3
    _close(ds, sf.grad, what="mse grad")


# ------------------------------------------------------------------------------- attention
def _attn_ref(qkv, cu, H, D, window, scale):
    """Dense masked softmax attention in fp32; returns out [T, H*D] and leaves autograd on."""
    T = qkv.shape[0]
    q, kk, v = qkv.view(T, 3, H, D).unbind(1)
    seq_id = torch.zeros(T, dtype=torch.long, device=qkv.device)
    for i in range(len(cu) - 1):
        seq_id[cu[i]:cu[i + 1]] = i
    pos = torch.arange(T, device=qkv.device)
    mask = seq_id[:, None] == seq_id[None, :]
    if window >= 0:
        mask &= (pos[:, None] - pos[None, :]).abs() <= window
    s = torch.einsum("thd,shd->hts", q, kk) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, v).reshape(T, H * D)


@pytest.mark.parametrize("lens", [[128], [50, 200, 6, 300, 77], [512, 512], [1, 2, 3, 700, 20, 20, 20, 20, 190]])
@pytest.mark.parametrize("window", [-1, 64])
def test_attention_fwd_bwd(lens, window, cuda_status):
    k = _k()
    H, D = 4, 64
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    qkv = _randn(T, 3 * H * D)
    scale = D ** -0.5
    ss, se = k.seq_bounds(cu_t, T)
    out, lse = k.fa_fwd(qkv, ss, se, H, D, window, scale)
    qf = qkv.float().requires_grad_(True)
    ref = _attn_ref(qf, cu, H, D, window, scale)
    _close(out, ref, what=f"attn fwd {lens} w={window}")
    dout = _randn(T, H * D)
    ref.backward(dout.float())
    dqkv = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale)
    _close(dqkv, qf.grad, rtol=3e-2, atol=3e-2, what=f"attn bwd {lens} w={window}")


def test_attention_determinism_and_big(cuda_status):
    k = _k()
    H, D = 16, 64
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(20, 513, (60,), generator=g).tolist()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    qkv = _randn(T, 3 * H * D)
    ss, se = k.seq_bounds(cu_t, T)
    o1, l1 = k.fa_fwd(qkv, ss, se, H, D, -1, 0.125)
    o2, l2 = k.fa_fwd(qkv, ss, se, H, D, -1, 0.125)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    # compare one head against the dense oracle
    sub = qkv.view(T, 3, H, D)[:, :, :2].reshape(T, 3 * 2 * D).contiguous()
    ref = _attn_ref(sub.float(), cu, 2, D, -1, 0.125)
    _close(o1.view(T, H, D)[:, :2].reshape(T, 2 * D), ref, what="attn big")


def test_gemm_rope_epilogue_and_attention_rope_backward(cuda_status):
    """RoPE fused into the QKV GEMM epilogue and un-done inside the attention backward must equal
    the separate rope kernel around the plain GEMM / attention."""
    k = _k()
    H, D, C = 4, 64, 256
    lens = [50, 200, 6, 300, 77]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32).cuda()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(512, device="cuda").float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    x, w = _randn(T, C), _randn(3 * H * D, C, scale=0.1)
    fused = k.gemm(x, w, epi=k.EPI_ROPE, rope=(pos, cos, sin, 2 * H * D))
    ref = k.gemm(x, w)
    k.rope_(ref, pos, cos, sin, H, D)
    _close(fused, ref, what="gemm rope epilogue")
    ss, se = k.seq_bounds(cu_t, T)
    out, lse = k.fa_fwd(ref, ss, se, H, D, -1, 0.125)
    dout = _randn(T, H * D)
    d_plain = k.fa_bwd(ref, out, dout, lse, ss, se, H, D, -1, 0.125)
    k.rope_(d_plain, pos, cos, sin, H, D, backward=True)
    d_fused = k.fa_bwd(ref, out, dout, lse, ss, se, H, D, -1, 0.125, rope=(pos, cos, sin))
    _close(d_fused, d_plain, rtol=3e-2, atol=3e-2, what="attention backward with fused inverse rope")


def test_linear_relu_epilogue(cuda_status):
    """ReLU in the GEMM epilogue (teacher feed-forward): forward under no_grad and forward + backward."""
    from nanoplm_b200.ops import functional as ops
    torch.manual_seed(0)
    x = torch.randn(777, 256, device="cuda").to(BF)
    w = (torch.randn(512, 256, device="cuda") * 0.1).to(BF)
    ref = torch.relu(x.float() @ w.float().t())
    with torch.no_grad():
        y = ops.linear(x, w, act="relu")
    assert (y.float() - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 0.02
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    gy = torch.randn(777, 512, device="cuda").to(BF)
    ops.linear(xg, wg, act="relu").backward(gy)
    x32, w32 = x.float().requires_grad_(True), w.float().requires_grad_(True)
    torch.relu(x32 @ w32.t()).backward(gy.float())
    assert (xg.grad.float() - x32.grad).abs().max().item() < 0.05 * x32.grad.abs().max().item()
    assert (wg.grad.float() - w32.grad).abs().max().item() < 0.05 * w32.grad.abs().max().item()


@pytest.mark.parametrize("form", ["store", "add", "swiglu", "rope", "dgrad", "wgrad"])
def test_gemm_cta_pair_matches_fp32(form, cuda_status):
    """The cta_group::2 GEMM (two SMs per 256 x 256 tile) against fp32 matmul, in every form the
    training step uses; shapes with partial tiles in M and N."""
    from nanoplm_b200.ops import kernels as K
    torch.manual_seed(0)
    dev = "cuda"
    M, N, Kd = 1000, 768, 320
    x = torch.randn(M, Kd, device=dev).to(BF)
    w = (torch.randn(N, Kd, device=dev) * 0.1).to(BF)
    ref = x.float() @ w.float().t()
    tol = lambda r: 0.02 * r.abs().max().item() + 0.02
    if form == "store":
        y = K.gemm(x, w, bn=256, pair=True)
        assert (y.float() - ref).abs().max().item() < tol(ref)
    elif form == "add":
        res = torch.randn(M, N, device=dev).to(BF)
        y = K.gemm(x, w, epi=K.EPI_ADD, aux=res, bn=256, pair=True)
        assert (y.float() - (ref + res.float())).abs().max().item() < tol(ref)
    elif form == "swiglu":
        pre = torch.empty(M, N, dtype=BF, device=dev)
        y = K.gemm(x, w, epi=K.EPI_SWIGLU, aux=pre, bn=256, pair=True)
        z = ref.to(BF).float()
        want = torch.nn.functional.silu(z[:, N // 2:]) * z[:, :N // 2]
        assert (pre.float() - z).abs().max().item() < tol(z)
        assert (y.float() - want).abs().max().item() < tol(want)
    elif form == "rope":
        H, D = N // 64 // 3, 64                      # q and k parts rotated, v untouched
        pos = torch.randint(0, 100, (M,), device=dev, dtype=torch.int32)
        inv = 1.0 / (10000.0 ** (torch.arange(0, 32, device=dev).float() / 32))
        ang = torch.arange(128, device=dev).float()[:, None] * inv[None, :]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        y = K.gemm(x, w, epi=K.EPI_ROPE, rope=(pos, cos, sin, 2 * H * D), bn=256, pair=True).float()
        want = ref.clone().view(M, N // 64, 64)
        c, s_ = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
        a, b = want[:, :2 * H, :32].clone(), want[:, :2 * H, 32:].clone()
        want[:, :2 * H, :32] = a * c - b * s_
        want[:, :2 * H, 32:] = b * c + a * s_
        assert (y - want.view(M, N)).abs().max().item() < tol(ref)
    elif form == "dgrad":
        dy = torch.randn(M, N, device=dev).to(BF)
        dx = K.gemm(dy, w[:, :256].contiguous(), b_mn=True, bn=256, pair=True)      # [M, 256]
        want = dy.float() @ w[:, :256].float()
        assert (dx.float() - want).abs().max().item() < tol(want)
    else:
        T = 4096 + 64
        dy = torch.randn(T, 512, device=dev).to(BF)
        xx = torch.randn(T, 256, device=dev).to(BF)
        acc = torch.ones(512, 256, dtype=torch.float32, device=dev)
        K.gemm(dy, xx, a_mn=True, b_mn=True, epi=K.EPI_ATOMIC_F32, out=acc, splits=3, bn=256, pair=True)
        want = 1.0 + dy.float().t() @ xx.float()
        assert (acc - want).abs().max().item() < 0.01 * want.abs().max().item() + 0.05


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("shape", [(512, 256, 4096 + 64), (960, 768, 20000), (3072, 1024, 8192)])
def test_gemm_stream_k_wgrad_matches_fp32(shape, pair, cuda_status):
    """splits=0 cuts tiles x k-blocks into one contiguous range per CTA (or CTA pair): every piece
    is added atomically, so the sum equals the plain product whatever the cut points are."""
    from nanoplm_b200.ops import kernels as K
    torch.manual_seed(1)
    n_out, k_in, T = shape
    dy = torch.randn(T, n_out, device="cuda").to(BF)
    xx = torch.randn(T, k_in, device="cuda").to(BF)
    acc = torch.ones(n_out, k_in, dtype=torch.float32, device="cuda")
    K.gemm(dy, xx, a_mn=True, b_mn=True, epi=K.EPI_ATOMIC_F32, out=acc, splits=0, bn=256, pair=pair)
    want = 1.0 + dy.float().t() @ xx.float()
    assert (acc - want).abs().max().item() < 0.01 * want.abs().max().item() + 0.05


@pytest.mark.parametrize("T,C,I", [(1000, 256, 512), (333, 128, 192), (4096, 1024, 2048)])
def test_swiglu_backward_epilogue_and_fused_mlp(T, C, I, cuda_status):
    """The gradient of the SwiGLU pre-activations computed in the epilogue of the dL/dh GEMM
    against fp32 autograd, and the fused MLP node against the two-linear composition."""
    from nanoplm_b200.ops import functional as ops
    from nanoplm_b200.ops import kernels as K
    torch.manual_seed(5)
    x = _randn(T, C)
    w_in = _randn(2 * I, C, scale=C ** -0.5)
    w_out = _randn(C, I, scale=I ** -0.5)
    res = _randn(T, C)
    dy = _randn(T, C)
    # epilogue alone
    pre = (x.float() @ w_in.float().t()).to(BF)
    dpre = K.gemm(dy, w_out, b_mn=True, epi=K.EPI_SWIGLU_BWD, aux=pre)
    assert dpre.shape == (T, 2 * I)
    p32 = pre.float().requires_grad_(True)
    v, g = p32.chunk(2, dim=-1)
    (F.silu(g) * v).backward(dy.float() @ w_out.float())
    _close(dpre, p32.grad, what="swiglu bwd epilogue")
    # fused node, forward and all four gradients
    xs, wi, wo, rs = (t.clone().requires_grad_(True) for t in (x, w_in, w_out, res))
    out = ops.mlp_swiglu(xs, wi, wo, rs)
    out.backward(dy)
    x32, wi32, wo32, r32 = (t.float().requires_grad_(True) for t in (x, w_in, w_out, res))
    v, g = (x32 @ wi32.t()).chunk(2, dim=-1)
    ref = (F.silu(g) * v) @ wo32.t() + r32
    ref.backward(dy.float())
    _close(out, ref, what="fused mlp out")
    _close(xs.grad, x32.grad, rtol=3e-2, atol=3e-2, what="fused mlp dx")
    _close(wi.grad, wi32.grad, rtol=3e-2, atol=3e-2, what="fused mlp dw_in")
    _close(wo.grad, wo32.grad, rtol=3e-2, atol=3e-2, what="fused mlp dw_out")
    _close(rs.grad, r32.grad, what="fused mlp dres")


@pytest.mark.parametrize("T,H", [(1000, 4), (333, 2), (4096, 16)])
def test_dgrad_with_delta_epilogue_and_fused_attention_node(T, H, cuda_status):
    """dO = dy @ W with rowsum(dO * O) per head from the same epilogue against fp32, and the fused
    attention + output projection node against the two separate ops (same kernels otherwise)."""
    from nanoplm_b200.ops import functional as ops
    from nanoplm_b200.ops import kernels as K
    torch.manual_seed(7)
    D, C = 64, H * 64
    dy = _randn(T, C)
    w = _randn(C, C, scale=C ** -0.5)
    o = _randn(T, C)
    delta = torch.full((H, T), 7.0, dtype=torch.float32, device="cuda")
    dout = K.gemm_dgrad_delta(dy, w, o, delta)
    ref = dy.float() @ w.float()
    _close(dout, ref, what="dgrad")
    want = (dout.float() * o.float()).view(T, H, D).sum(-1).t()
    assert (delta - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())
    # fused node vs attention_varlen + linear
    lens = [T // 3, T // 5, T - T // 3 - T // 5]
    cu = torch.tensor([0, lens[0], lens[0] + lens[1], T], dtype=torch.int32, device="cuda")
    ss, se = ops.seq_bounds(cu, T)
    qkv = _randn(T, 3 * C, scale=0.5)
    res = _randn(T, C)
    for window in (-1, 64):
        grads = []
        outs = []
        for fused in (True, False):
            q, ww, r = (t.clone().requires_grad_(True) for t in (qkv, w, res))
            if fused:
                y = ops.attention_out_proj(q, ww, r, ss, se, H, D, window, D ** -0.5)
            else:
                y = ops.linear(ops.attention_varlen(q, ss, se, H, D, window, D ** -0.5), ww, residual=r)
            y.backward(dy)
            outs.append(y)
            grads.append((q.grad, ww.grad, r.grad))
        assert torch.equal(outs[0], outs[1])
        for a, b, name in zip(grads[0], grads[1], ("dqkv", "dw", "dres")):
            _close(a, b, rtol=2e-2, atol=2e-2, what=f"fused attention node {name} window={window}")
