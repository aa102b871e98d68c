"""CPU restatements behind the fused autograd nodes: off the GPU the fused entry points must be
plain compositions of the basic ops, and Muon's batched Newton-Schulz must treat every matrix of a
stack on its own."""
import torch
import torch.nn.functional as F


def test_mlp_swiglu_is_the_two_linear_composition_on_cpu():
    from nanoplm_b200.ops import functional as ops
    torch.manual_seed(0)
    x = torch.randn(37, 48, requires_grad=True)
    wi = (torch.randn(2 * 64, 48) * 0.1).requires_grad_(True)
    wo = (torch.randn(48, 64) * 0.1).requires_grad_(True)
    res = torch.randn(37, 48, requires_grad=True)
    y = ops.mlp_swiglu(x, wi, wo, res)
    v, g = F.linear(x, wi).chunk(2, dim=-1)
    ref = F.linear(F.silu(g) * v, wo) + res
    assert torch.allclose(y, ref, atol=1e-6)
    y.sum().backward()
    assert x.grad is not None and wi.grad is not None and wo.grad is not None and res.grad is not None


def test_attention_out_proj_is_attention_then_linear_on_cpu():
    from nanoplm_b200.ops import functional as ops
    torch.manual_seed(1)
    T, H, D = 50, 2, 16
    qkv = torch.randn(T, 3 * H * D, requires_grad=True)
    w = (torch.randn(H * D, H * D) * 0.2).requires_grad_(True)
    res = torch.randn(T, H * D)
    cu = torch.tensor([0, 20, 50], dtype=torch.int32)
    ss, se = ops.seq_bounds(cu, T)
    for window in (-1, 4):
        y = ops.attention_out_proj(qkv, w, res, ss, se, H, D, window, D ** -0.5)
        ref = F.linear(ops.attention_varlen(qkv, ss, se, H, D, window, D ** -0.5), w) + res
        assert torch.allclose(y, ref, atol=1e-6)
    # tokens of the first sequence must not see the second one
    y1 = ops.attention_out_proj(qkv[:20].detach(), w.detach(), res[:20], ss[:20], se[:20], H, D, -1, D ** -0.5)
    y_full = ops.attention_out_proj(qkv.detach(), w.detach(), res, ss, se, H, D, -1, D ** -0.5)
    assert torch.allclose(y1, y_full[:20], atol=1e-5)


def test_batched_newton_schulz_treats_matrices_independently():
    from nanoplm_b200.parallel.muon import POLAR_EXPRESS, orthogonalize, orthogonalize_batched
    torch.manual_seed(2)
    G = torch.randn(3, 24, 40) * torch.tensor([0.01, 1.0, 50.0])[:, None, None]
    both = orthogonalize_batched(G, POLAR_EXPRESS)
    for i in range(3):
        assert torch.allclose(both[i], orthogonalize(G[i], POLAR_EXPRESS), atol=1e-5)
        sv = torch.linalg.svdvals(both[i])
        assert 0.95 < sv.min() and sv.max() < 1.05
    tall = orthogonalize_batched(G.transpose(1, 2).contiguous(), POLAR_EXPRESS)
    assert tall.shape == (3, 40, 24)
    assert torch.allclose(tall, both.transpose(1, 2), atol=1e-5)
