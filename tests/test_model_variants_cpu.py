"""The additive encoder variants on the CPU restatements: varlen depthwise convolution, hyper-connections
(n residual streams mixed by a Sinkhorn-projected matrix), MoE layers and RMSNorm. None of them has a
reference counterpart, so the checks are properties: no leakage across sequence boundaries, a doubly
stochastic stream mix, routing statistics, gradients on every parameter, and a loss that falls."""
import torch

from nanoplm_b200.config.schema import ModelConfig
from nanoplm_b200.data.tokenizer import ProtTokenizer
from nanoplm_b200.models.encoder import ProtEncoderMLM
from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine

GEOM = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=2, max_position_embeddings=64)


def _batch(seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(4, 24, (90,), generator=g)
    cu = torch.tensor([0, 25, 60, 90], dtype=torch.int32)
    lab = torch.full((90,), -100)
    lab[::3] = ids[::3]
    return ids, cu, lab


def _model(**kw):
    torch.manual_seed(0)
    m = ProtEncoderMLM(ModelConfig(**GEOM, **kw), ProtTokenizer())
    with torch.no_grad():                       # the output projections start at zero: make every path matter
        for n, p in m.named_parameters():
            if n.endswith("Wo.weight") or "experts_Wo" in n:
                p.normal_(0, 0.05)
    return m


def test_variants_train_and_every_parameter_gets_a_gradient():
    ids, cu, lab = _batch()
    for kw in (dict(conv_kernel_size=7, conv_bias=True), dict(mhc_streams=4), dict(norm_type="rmsnorm"),
               dict(moe={"num_experts": 4, "top_k": 2, "expert_intermediate_size": 16, "every_n_layers": 2}),
               dict(conv_kernel_size=7, mhc_streams=4, norm_type="rmsnorm",
                    moe={"num_experts": 4, "top_k": 2, "expert_intermediate_size": 16, "every_n_layers": 2})):
        m = _model(**kw)
        out = m(input_ids=ids, cu_seqlens=cu, labels=lab)
        out["loss"].backward()
        missing = [n for n, p in m.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
        assert not missing, (kw, missing)
        if "moe" in kw:
            assert out["aux_loss"] is not None and float(out["aux_loss"]) > 0
            assert float(m.model.layers[1].mlp.router.weight.grad.abs().sum()) > 0
        m.zero_grad(set_to_none=True)
        eng = ShardedEngine(m, AdamWHyper(lr=3e-3), torch.device("cpu"))
        losses = []
        for _ in range(12):
            loss = m(input_ids=ids, cu_seqlens=cu, labels=lab)["loss"]
            loss.backward()
            eng.step(3e-3, 1)
            losses.append(float(loss.detach()))
        assert losses[-1] < losses[0] - 0.05, (kw, losses)


def test_conv_and_attention_do_not_leak_across_sequence_boundaries():
    ids, cu, _ = _batch()
    m = _model(conv_kernel_size=7, mhc_streams=4).eval()
    with torch.no_grad():
        base = m(input_ids=ids, cu_seqlens=cu)["logits"]
        other = ids.clone()
        other[25:60] = torch.randint(4, 24, (35,), generator=torch.Generator().manual_seed(9))     # the middle sequence only
        changed = m(input_ids=other, cu_seqlens=cu)["logits"]
    assert torch.equal(base[:25], changed[:25]) and torch.equal(base[60:], changed[60:])
    assert not torch.allclose(base[25:60], changed[25:60])


def test_hyper_connection_mix_is_doubly_stochastic_and_starts_as_a_plain_residual():
    from nanoplm_b200.models.mhc import HyperConnection, sinkhorn
    torch.manual_seed(0)
    R = sinkhorn(torch.randn(5, 4, 4), 30)
    assert torch.allclose(R.sum(-1), torch.ones(5, 4), atol=1e-4) and torch.allclose(R.sum(-2), torch.ones(5, 4), atol=1e-4)
    assert bool((R > 0).all())
    hc = HyperConnection(32, 4, sinkhorn_iters=5)
    X = torch.randn(10, 4, 32)
    h, state = hc.read(X)
    assert h.shape == (10, 32)
    Xn = hc.write(X, torch.zeros(10, 32), state)
    assert Xn.shape == X.shape
    # writing a zero branch output only mixes the streams: their sum per token is preserved by a doubly stochastic mix
    assert torch.allclose(Xn.sum(dim=1), X.sum(dim=1), atol=1e-4)


def test_moe_routing_statistics():
    from nanoplm_b200.models.moe import route_topk
    torch.manual_seed(0)
    logits = torch.randn(200, 8)
    gates, experts, aux = route_topk(logits, 2)
    assert gates.shape == experts.shape == (200, 2)
    assert torch.allclose(gates.sum(-1), torch.ones(200), atol=1e-6)            # renormalised over the chosen experts
    assert bool((experts[:, 0] != experts[:, 1]).all()) and int(experts.max()) < 8
    top = logits.softmax(-1).topk(2, dim=-1).indices
    assert torch.equal(experts.sort(-1).values, top.sort(-1).values)
    assert float(aux) >= 1.0 - 1e-3                                              # E * sum f_e P_e is 1 for a perfectly even router
    even = route_topk(torch.zeros(64, 8) + torch.arange(8) * 1e-6, 2)[2]
    assert float(even) > 0
