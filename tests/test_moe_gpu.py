"""GPU tests of the mixture-of-experts kernels (router, plan, push / pull, grouped tcgen05 GEMM)
against plain PyTorch fp32 restatements of the same operations."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _route_ref(logits32: torch.Tensor, k: int, experts=None):
    """Softmax router. With `experts` given the selection is taken from there (bf16 logits have
    exact ties, which top-k implementations may break differently)."""
    probs = torch.softmax(logits32, dim=-1)
    if experts is None:
        g, e = torch.topk(probs, k, dim=-1)
    else:
        e = experts.long()
        g = torch.gather(probs, 1, e)
    gates = g / g.sum(-1, keepdim=True)
    E = logits32.shape[1]
    counts = torch.bincount(e.reshape(-1), minlength=E).float()
    aux = E * ((counts / e.numel()) * probs.mean(0)).sum()
    return probs, gates, e, counts, aux


@pytest.mark.parametrize("T,E,k", [(1000, 8, 2), (4096, 64, 2), (333, 40, 4)])
def test_router_topk_and_backward(T, E, k, cuda_status):
    from nanoplm_b200.ops import moe as M
    torch.manual_seed(0)
    dev = torch.device("cuda:0")
    logits = (torch.randn(T, E, device=dev) * 2).to(BF)
    probs, gates, experts, probsum, counts = M.router_topk(logits, k)
    l32 = logits.float().requires_grad_(True)
    top_vals = torch.topk(torch.softmax(logits.float(), -1), k, dim=-1).values
    p_ref, g_ref, e_ref, c_ref, aux_ref = _route_ref(l32, k, experts)
    assert torch.allclose(torch.gather(p_ref.detach(), 1, experts.long()), top_vals, atol=1e-6)
    assert all(len(set(row)) == k for row in experts[:64].tolist())
    assert torch.allclose(probs, p_ref.detach(), atol=1e-5)
    assert torch.allclose(gates, g_ref.detach(), atol=1e-5)
    assert torch.equal(counts.float(), c_ref)
    assert torch.allclose(probsum, p_ref.detach().sum(0), rtol=1e-4, atol=1e-3)
    # backward through the gates and the balance loss
    d_gates = torch.randn(T, k, device=dev)
    (g_ref * d_gates).sum().add(0.37 * aux_ref).backward()
    f = c_ref / float(T * k)
    aux_grad = (0.37 * E / T * f).contiguous()
    dl = M.router_bwd(probs, gates, experts, d_gates, aux_grad)
    err = (dl.float() - l32.grad).abs().max().item()
    assert err < 2e-2 * max(1.0, l32.grad.abs().max().item()), err


@pytest.mark.parametrize("T,E,k", [(1000, 8, 2), (5000, 64, 2)])
def test_plan_layout(T, E, k, cuda_status):
    from nanoplm_b200.ops import moe as M
    torch.manual_seed(1)
    dev = torch.device("cuda:0")
    experts = torch.randint(0, E, (T, k), device=dev, dtype=torch.int32)
    if E == 64:
        experts[experts == 5] = 6          # one expert without any token
    comm = M.MoEComm(64, E, k)
    plan = M.make_plan(comm, experts)
    torch.cuda.synchronize()
    flat = experts.reshape(-1).cpu()
    pos = plan.pos_of.cpu()
    off = plan.group_off.cpu()
    counts = torch.bincount(flat.long(), minlength=E)
    exp_off = torch.zeros(E + 1, dtype=torch.long)
    exp_off[1:] = torch.cumsum((counts + 127) // 128 * 128, 0)
    assert torch.equal(off.long(), exp_off)
    for e in range(E):
        idx = (flat == e).nonzero().flatten()
        assert torch.equal(pos[idx].long(), exp_off[e] + torch.arange(len(idx)))
    tg = plan.tile_group.cpu()
    for tile in range(len(tg)):
        row = tile * 128
        want = -1
        if row < exp_off[-1]:
            want = int((exp_off[1:] > row).nonzero()[0])
        assert tg[tile] == want, (tile, tg[tile], want)
    assert torch.equal(plan.pad_lo.cpu().long(), exp_off[:-1] + counts)
    assert torch.equal(plan.pad_hi.cpu().long(), exp_off[1:])


def _random_plan(T, E, k, C, dev):
    from nanoplm_b200.ops import moe as M
    experts = torch.randint(0, E, (T, k), device=dev, dtype=torch.int32)
    comm = M.MoEComm(C, E, k)
    return M.make_plan(comm, experts), experts


@pytest.mark.parametrize("T,E,C,N", [(1500, 8, 256, 512), (3000, 16, 512, 384)])
def test_grouped_gemm_forms(T, E, C, N, cuda_status):
    from nanoplm_b200.ops import kernels as K
    from nanoplm_b200.ops import moe as M
    torch.manual_seed(2)
    dev = torch.device("cuda:0")
    k = 2
    plan, experts = _random_plan(T, E, k, C, dev)
    P = plan.cap
    off = plan.group_off.cpu().tolist()
    a = torch.randn(P, C, device=dev).to(BF)
    W = (torch.randn(E, N, C, device=dev) * 0.05).to(BF)
    out = M.gemm_grouped(a, W, plan.tile_group)
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        if r1 > r0:
            ref = a[r0:r1].float() @ W[e].float().t()
            assert (out[r0:r1].float() - ref).abs().max().item() < 0.06 * ref.abs().max().item() + 0.02
    # SwiGLU epilogue (N must be even: value rows then gate rows)
    pre = torch.empty(P, N, dtype=BF, device=dev)
    h = M.gemm_grouped(a, W, plan.tile_group, epi=K.EPI_SWIGLU, aux=pre)
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        if r1 > r0:
            z = (a[r0:r1].float() @ W[e].float().t()).to(BF).float()
            ref = torch.nn.functional.silu(z[:, N // 2:]) * z[:, :N // 2]
            assert (h[r0:r1].float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 0.02
            assert (pre[r0:r1].float() - z).abs().max().item() < 0.05 * z.abs().max().item() + 0.02
    # data gradient form: dY [P,N] x W[e] [N,C]
    dy = torch.randn(P, N, device=dev).to(BF)
    dx = M.gemm_grouped(dy, W, plan.tile_group, b_mn=True)
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        if r1 > r0:
            ref = dy[r0:r1].float() @ W[e].float()
            assert (dx[r0:r1].float() - ref).abs().max().item() < 0.06 * ref.abs().max().item() + 0.02
    # weight gradient form, accumulated on top of existing values
    acc = torch.ones(E, N, C, dtype=torch.float32, device=dev)
    M.gemm_grouped_wgrad(dy, a, plan.group_off, acc)
    for e in range(E):
        r0, r1 = off[e], off[e + 1]
        ref = 1.0 + dy[r0:r1].float().t() @ a[r0:r1].float()
        assert (acc[e] - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 0.05


def _moe_oracle(x32, logits32, Wi32, Wo32, k, experts):
    """fp32 restatement: softmax router, top-k, renormalised gates, SwiGLU experts."""
    probs, gates, e, counts, aux = _route_ref(logits32, k, experts)
    I = Wo32.shape[2]
    y = torch.zeros_like(x32)
    for s in range(k):
        for ex in range(Wi32.shape[0]):
            sel = (e[:, s] == ex).nonzero().flatten()
            if len(sel) == 0:
                continue
            z = x32[sel] @ Wi32[ex].t()
            hh = torch.nn.functional.silu(z[:, I:]) * z[:, :I]
            y = y.index_add(0, sel, (hh @ Wo32[ex].t()) * gates[sel, s:s + 1])
    return y, aux


@pytest.mark.parametrize("T,E,k,C,I", [(1111, 8, 2, 256, 128), (2048, 16, 1, 128, 256)])
def test_moe_mlp_forward_backward(T, E, k, C, I, cuda_status):
    from nanoplm_b200.ops import moe as M
    torch.manual_seed(3)
    dev = torch.device("cuda:0")
    x = torch.randn(T, C, device=dev).to(BF).requires_grad_(True)
    logits = (torch.randn(T, E, device=dev) * 1.5).to(BF).requires_grad_(True)
    Wi = (torch.randn(E, 2 * I, C, device=dev) * 0.06).to(BF).requires_grad_(True)
    Wo = (torch.randn(E, C, I, device=dev) * 0.06).to(BF).requires_grad_(True)
    comm = M.MoEComm(C, E, k)
    y, aux = M.moe_mlp(x, logits, Wi, Wo, k, comm)
    gy = torch.randn(T, C, device=dev).to(BF)
    ((y.float() * gy.float()).sum() + 0.5 * aux).backward()
    x32 = x.detach().float().requires_grad_(True)
    l32 = logits.detach().float().requires_grad_(True)
    Wi32 = Wi.detach().float().requires_grad_(True)
    Wo32 = Wo.detach().float().requires_grad_(True)
    experts = M.router_topk(logits.detach(), k)[2]
    y_ref, aux_ref = _moe_oracle(x32, l32, Wi32, Wo32, k, experts)
    ((y_ref * gy.float()).sum() + 0.5 * aux_ref).backward()
    torch.cuda.synchronize()

    def close(a, b, tol, what):
        err = (a.float() - b.float()).abs().max().item()
        ref = b.float().abs().max().item()
        assert err <= tol * ref + 1e-3, (what, err, ref)

    close(y, y_ref, 0.04, "y")
    assert abs(aux.item() - aux_ref.item()) < 1e-3
    close(x.grad, x32.grad, 0.05, "dx")
    close(logits.grad, l32.grad, 0.06, "dlogits")
    close(Wi.grad, Wi32.grad, 0.05, "dWi")
    close(Wo.grad, Wo32.grad, 0.05, "dWo")


def test_grouped_gemm_gated_by_arrival_counters_matches_ungated(cuda_status):
    """The arrival-gated grouped GEMM (counters already at their expected values, as after a finished
    dispatch) gives the bits of the ungated one; counters ABOVE the expectation also pass."""
    from nanoplm_b200.ops import moe as M
    torch.manual_seed(4)
    dev = torch.device("cuda:0")
    T, E, k, C, N = 3000, 8, 2, 256, 512
    plan, _ = _random_plan(T, E, k, C, dev)
    P = plan.cap
    a = torch.randn(P, C, device=dev).to(BF)
    W = (torch.randn(E, N, C, device=dev) * 0.05).to(BF)
    ref = M.gemm_grouped(a, W, plan.tile_group)
    tiles = P // 128
    expect = torch.randint(0, 129, (tiles,), device=dev, dtype=torch.int32)
    for extra in (0, 5):
        arrive = (expect + extra).contiguous()
        out = M.gemm_grouped(a, W, plan.tile_group, arrive=arrive, expect=expect)
        rows = (plan.tile_group >= 0).repeat_interleave(128)
        assert torch.equal(out[rows], ref[rows])
    with pytest.raises(ValueError):
        M.gemm_grouped(a, W, plan.tile_group, arrive=expect)
