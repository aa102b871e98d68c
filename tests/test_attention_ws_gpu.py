"""Warp-specialised varlen attention (attention_ws.cu) against a dense fp32 masked-softmax oracle
and against the single-role kernels, on a sweep that includes one-token, odd and tile-straddling
flat lengths, empty sequences and both window settings."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _k():
    from nanoplm_b200.ops import kernels
    return kernels


def _oracle(qkv, cu, H, D, window, scale):
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
    lse = torch.logsumexp(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, v).reshape(T, H * D), lse


def _cu(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return cu


SWEEP = [
    [1], [7], [129], [128], [255, 1], [256], [257],
    [50, 200, 6, 300, 77],
    [512, 512],
    [1, 2, 3, 700, 20, 20, 20, 20, 190],
    [0, 5, 0, 0, 130, 0, 64, 0],          # empty sequences, as the static collator emits them
    [4097],
    [300] * 9 + [41],
]


@pytest.mark.parametrize("lens", SWEEP, ids=lambda l: "-".join(map(str, l))[:40])
@pytest.mark.parametrize("window", [-1, 64])
def test_ws_forward_matches_oracle(lens, window, cuda_status):
    k = _k()
    H, D = 4, 64
    cu = _cu(lens)
    T = cu[-1]
    torch.manual_seed(T + window)
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ss, se = k.seq_bounds(cu_t, T)
    scale = D ** -0.5
    out, lse = k.fa_fwd(qkv, ss, se, H, D, window, scale, impl="ws")
    ref, ref_lse = _oracle(qkv.float(), cu, H, D, window, scale)
    # bf16 output of an average of unit-variance values: error bound 2^-8 relative + P rounding
    err = (out.float() - ref).abs().max().item()
    assert err <= 2.5e-2, f"forward {lens} w={window}: max err {err}"
    lerr = (lse - ref_lse).abs().max().item()
    assert lerr <= 2e-3 * max(1.0, ref_lse.abs().max().item()), f"lse {lens} w={window}: {lerr}"
    old, old_lse = k.fa_fwd(qkv, ss, se, H, D, window, scale, impl="single")
    assert (out.float() - old.float()).abs().max().item() <= 2e-2
    assert (lse - old_lse).abs().max().item() <= 2e-3 * max(1.0, ref_lse.abs().max().item())


def test_ws_forward_is_deterministic_and_handles_a_full_batch(cuda_status):
    k = _k()
    H, D = 16, 64
    g = torch.Generator().manual_seed(1)
    lens = torch.randint(20, 513, (70,), generator=g).tolist()
    cu = _cu(lens)
    T = cu[-1]
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ss, se = k.seq_bounds(cu_t, T)
    for window in (-1, 64):
        o1, l1 = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        o2, l2 = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        assert torch.equal(o1, o2) and torch.equal(l1, l2)
        # a limited grid walks more items per CTA: same result
        o3, l3 = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws", max_ctas=7)
        assert torch.equal(o1, o3) and torch.equal(l1, l3)
        sub = qkv.view(T, 3, H, D)[:, :, 3:5].reshape(T, 3 * 2 * D).contiguous()
        ref, _ = _oracle(sub.float(), cu, 2, D, window, 0.125)
        err = (o1.view(T, H, D)[:, 3:5].reshape(T, 2 * D).float() - ref).abs().max().item()
        assert err <= 2.5e-2, f"w={window}: {err}"


@pytest.mark.parametrize("lens", SWEEP, ids=lambda l: "-".join(map(str, l))[:40])
@pytest.mark.parametrize("window", [-1, 64])
def test_ws_backward_matches_autograd_of_the_oracle(lens, window, cuda_status):
    k = _k()
    H, D = 4, 64
    cu = _cu(lens)
    T = cu[-1]
    torch.manual_seed(3 * T + window)
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ss, se = k.seq_bounds(cu_t, T)
    scale = D ** -0.5
    out, lse = k.fa_fwd(qkv, ss, se, H, D, window, scale, impl="ws")
    qf = qkv.float().requires_grad_(True)
    ref, _ = _oracle(qf, cu, H, D, window, scale)
    ref.backward(dout.float())
    dqkv = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale, impl="ws")
    g = qf.grad
    # gradients are sums of up to a few hundred bf16-rounded products: bound relative to the
    # gradient's scale, plus the bf16 rounding of the stored value
    tol = 2.0 ** -6 * g.abs().max().item() + 2e-2
    err = (dqkv.float() - g).abs().max().item()
    assert err <= tol, f"backward {lens} w={window}: max err {err} (tol {tol})"
    old = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale, impl="single")
    assert (dqkv.float() - old.float()).abs().max().item() <= tol


def test_ws_backward_full_batch_with_fused_rope_and_limited_grid(cuda_status):
    k = _k()
    H, D = 16, 64
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(20, 513, (40,), generator=g).tolist()
    cu = _cu(lens)
    T = cu[-1]
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32).cuda()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(512, device="cuda").float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    ss, se = k.seq_bounds(cu_t, T)
    for window in (-1, 64):
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        a = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="ws")
        b = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="single")
        c = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="ws",
                     max_ctas=5)
        scale_ = b.float().abs().max().item()
        assert (a.float() - b.float()).abs().max().item() <= 2.0 ** -6 * scale_ + 2e-2
        assert (a.float() - c.float()).abs().max().item() <= 2.0 ** -6 * scale_ + 2e-2
        # dK and dV do not go through atomics: bitwise equal whatever the grid
        HD = H * D
        assert torch.equal(a[:, HD:], c[:, HD:])


def test_ws_backward_dk_dv_are_bitwise_reproducible(cuda_status):
    """dK and dV accumulate in TMEM in a fixed order: two runs give identical bits. (dQ is summed
    over key tiles with fp32 atomics in the default mode and may differ in the last bits.)"""
    k = _k()
    H, D = 8, 64
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(20, 513, (30,), generator=g).tolist()
    cu = _cu(lens)
    T = cu[-1]
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ss, se = k.seq_bounds(cu_t, T)
    HD = H * D
    for window in (-1, 64):
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        a = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl="ws")
        b = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, impl="ws")
        assert torch.equal(a[:, HD:], b[:, HD:])
        assert (a[:, :HD].float() - b[:, :HD].float()).abs().max().item() <= 2.0 ** -6 * a[:, :HD].float().abs().max().item()


DET_SWEEP = [[77], [128, 128], [300, 45, 512, 3], [512] * 3 + [20] * 7]


@pytest.mark.parametrize("lens", DET_SWEEP, ids=lambda l: "-".join(map(str, l))[:40])
@pytest.mark.parametrize("window", [-1, 64])
def test_ws_backward_deterministic_mode_matches_autograd_of_the_oracle(lens, window, cuda_status):
    """The query-stationary dQ launch against fp32 autograd, and dK / dV identical to the default mode."""
    k = _k()
    H, D = 4, 64
    cu = _cu(lens)
    T = cu[-1]
    torch.manual_seed(5 * T + window)
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    ss, se = k.seq_bounds(cu_t, T)
    scale = D ** -0.5
    out, lse = k.fa_fwd(qkv, ss, se, H, D, window, scale, impl="ws")
    qf = qkv.float().requires_grad_(True)
    ref, _ = _oracle(qf, cu, H, D, window, scale)
    ref.backward(dout.float())
    det = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale, impl="ws", deterministic=True)
    g = qf.grad
    tol = 2.0 ** -6 * g.abs().max().item() + 2e-2
    err = (det.float() - g).abs().max().item()
    assert err <= tol, f"deterministic backward {lens} w={window}: max err {err} (tol {tol})"
    dflt = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, scale, impl="ws", deterministic=False)
    HD = H * D
    assert torch.equal(det[:, HD:], dflt[:, HD:])


def test_ws_backward_deterministic_mode_is_bitwise_reproducible_with_rope(cuda_status):
    k = _k()
    H, D = 16, 64
    g = torch.Generator().manual_seed(9)
    lens = torch.randint(20, 513, (40,), generator=g).tolist()
    cu = _cu(lens)
    T = cu[-1]
    qkv = torch.randn(T, 3 * H * D, device="cuda").to(BF)
    dout = torch.randn(T, H * D, device="cuda").to(BF)
    cu_t = torch.tensor(cu, dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32).cuda()
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    fr = torch.outer(torch.arange(512, device="cuda").float(), inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    ss, se = k.seq_bounds(cu_t, T)
    for window in (-1, 64):
        out, lse = k.fa_fwd(qkv, ss, se, H, D, window, 0.125, impl="ws")
        a = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="ws",
                     deterministic=True)
        b = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="ws",
                     deterministic=True)
        c = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="ws",
                     deterministic=True, max_ctas=7)
        assert torch.equal(a, b)
        assert torch.equal(a, c)      # the grid changes which CTA runs an item, not the order inside it
        ref = k.fa_bwd(qkv, out, dout, lse, ss, se, H, D, window, 0.125, rope=(pos, cos, sin), impl="single")
        scale_ = ref.float().abs().max().item()
        assert (a.float() - ref.float()).abs().max().item() <= 2.0 ** -6 * scale_ + 2e-2
