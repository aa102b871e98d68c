"""GPU tests of the FP8 (e4m3, block128) kernels against PyTorch fp32 restatements: quantisation
(1 x 128 rows, 128 x 128 tiles, transposed forms), the tcgen05 fp8 GEMM with per-K-block promotion
(oracle: fp32 matmul of the de-quantised operands) and the autograd linear layer."""
import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _ref_quant_rows(x32: torch.Tensor):
    R, K = x32.shape
    xb = x32.view(R, K // 128, 128)
    s = xb.abs().amax(-1).clamp(min=1e-12) / 448.0
    q = (xb / s[..., None]).to(torch.float8_e4m3fn).float()
    return (q * s[..., None]).view(R, K), s


def test_quant_rows_matches_reference(cuda_status):
    from nanoplm_b200.ops import fp8
    torch.manual_seed(0)
    x = (torch.randn(777, 512, device="cuda") * 3).to(BF)
    qx = fp8.quant_rows(x)
    deq_ref, s_ref = _ref_quant_rows(x.float())
    assert torch.allclose(qx.scale.t(), s_ref, rtol=1e-6)
    deq = qx.dequantize()
    # identical scales; payload may differ by one e4m3 step where the division rounds differently
    assert (deq - deq_ref).abs().max().item() <= 0.07 * x.float().abs().max().item()
    assert ((deq - x.float()).abs() <= 0.0625 * x.float().abs() + 1e-3 * s_ref.max()).all()


@pytest.mark.parametrize("transpose,block", [(False, True), (True, True), (True, False)])
def test_quant_tile_forms(transpose, block, cuda_status):
    from nanoplm_b200.ops import fp8
    torch.manual_seed(1)
    R, K = 384, 256
    x = (torch.randn(R, K, device="cuda") * 2).to(BF)
    qx = fp8.quant_tile(x, transpose=transpose, block=block)
    deq = qx.dequantize()
    want = x.float().t() if transpose else x.float()
    assert deq.shape == want.shape
    assert ((deq - want).abs() <= 0.0625 * want.abs() + 0.02).all()
    if block:
        tiles = x.float().view(R // 128, 128, K // 128, 128).abs().amax(dim=(1, 3)) / 448.0   # [R/128, K/128]
        exp = tiles if transpose else tiles.t()
        assert torch.allclose(qx.scale, exp.contiguous(), rtol=1e-6)


@pytest.mark.parametrize("M,N,K,b_block", [(1000, 384, 512, True), (4096, 1024, 1024, True), (256, 640, 896, False)])
def test_gemm_fp8_matches_dequantised_matmul(M, N, K, b_block, cuda_status):
    from nanoplm_b200.ops import fp8
    torch.manual_seed(2)
    a = torch.randn(M, K, device="cuda").to(BF)
    b = (torch.randn(N, K, device="cuda") * 0.1).to(BF)
    qa = fp8.quant_rows(a)
    qb = fp8.quant_tile(b, transpose=False, block=True) if b_block else fp8.quant_rows(b)
    ref = qa.dequantize() @ qb.dequantize().t()
    out = fp8.gemm_fp8(qa, qb)
    err = (out.float() - ref).abs().max().item()
    assert err <= 0.01 * ref.abs().max().item() + 1e-2, err
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    fp8.gemm_fp8(qa, qb, out=acc, accumulate=True)
    assert (acc - 1.0 - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3


def test_fp8_linear_forward_backward(cuda_status):
    from nanoplm_b200.ops import fp8
    torch.manual_seed(3)
    T, Cin, Cout = 1024, 512, 768
    x = torch.randn(T, Cin, device="cuda").to(BF).requires_grad_(True)
    w = (torch.randn(Cout, Cin, device="cuda") * 0.05).to(BF).requires_grad_(True)
    gy = torch.randn(T, Cout, device="cuda").to(BF)
    fp8.invalidate_weight_cache()
    y = fp8.fp8_linear(x, w)
    y.backward(gy)
    x32, w32 = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    y_ref = x32 @ w32.t()
    y_ref.backward(gy.float())

    def rel(a, b):
        return (a.float() - b).norm().item() / b.norm().item()

    assert rel(y, y_ref) < 0.05
    assert rel(x.grad, x32.grad) < 0.05
    assert rel(w.grad, w32.grad) < 0.05


def test_encoder_trains_in_fp8(cuda_status):
    """A small encoder steps with every eligible linear layer in e4m3 and the loss goes down."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops import functional as ops
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from test_extras_gpu import _batch
    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256)
    model = ProtEncoderMLM(cfg, tok)
    eng = ShardedEngine(model, AdamWHyper(lr=2e-3), torch.device("cuda:0"))
    b = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in _batch(tok).items()}
    ops.set_fp8(True)
    try:
        losses = []
        for _ in range(8):
            out = model(**b)
            out["loss"].backward()
            eng.step(2e-3, 1)
            losses.append(out["loss"].item())
    finally:
        ops.set_fp8(False)
    assert losses[-1] < losses[0] - 0.05, losses
