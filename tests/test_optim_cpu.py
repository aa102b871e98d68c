"""Optimizer engines on CPU: sharded AdamW against torch.optim.AdamW + clip_grad_norm_, Muon /
NorMuon routing and orthogonalisation."""
import copy

import torch

from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig
from nanoplm_b200.data.tokenizer import ProtTokenizer
from nanoplm_b200.models.encoder import ProtEncoderMLM
from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine, use_weight_decay
from nanoplm_b200.parallel.muon import POLAR_EXPRESS, MuonEngine, orthogonalize


def _model():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                      max_position_embeddings=128)
    m = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for layer in m.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            layer.mlp.Wo.weight.normal_(0, 0.05)
    return m


def _batch():
    ids = torch.randint(4, 24, (150,))
    cu = torch.tensor([0, 40, 90, 150], dtype=torch.int32)
    lab = torch.full((150,), -100)
    lab[::4] = ids[::4]
    return dict(input_ids=ids, labels=lab, cu_seqlens=cu)


def test_engine_matches_torch_adamw_with_clipping():
    ref = _model()
    mine = copy.deepcopy(ref)
    decay = [p for n, p in ref.named_parameters() if use_weight_decay(n, p)]
    no_decay = [p for n, p in ref.named_parameters() if not use_weight_decay(n, p)]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.05}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=3e-3, betas=(0.9, 0.999), eps=1e-8)
    eng = ShardedEngine(mine, AdamWHyper(lr=3e-3, weight_decay=0.05, max_grad_norm=1.0), torch.device("cpu"))
    assert len(eng.slots) == len(decay) + len(no_decay)               # tied decoder weight counted once
    b = _batch()
    for step in range(5):
        for m in (ref, mine):
            for k in range(2):                                        # two micro-batches per step
                (m(**b)["loss"] / (2 if m is ref else 1)).backward()
        gn_ref = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        gn = eng.step(3e-3, grad_accum=2)
        assert abs(float(gn) - float(gn_ref)) / float(gn_ref) < 1e-4
    for (n1, p1), (n2, p2) in zip(ref.named_parameters(), mine.named_parameters()):
        assert n1 == n2 and torch.allclose(p1, p2, atol=2e-6), n1
    sd = eng.optimizer_state_dict()
    ref_sd = opt.state_dict()
    assert [len(g["params"]) for g in sd["param_groups"]] == [len(g["params"]) for g in ref_sd["param_groups"]]
    for i in ref_sd["state"]:
        assert torch.allclose(sd["state"][i]["exp_avg"], ref_sd["state"][i]["exp_avg"], atol=1e-7)
        assert float(sd["state"][i]["step"]) == float(ref_sd["state"][i]["step"])


def test_orthogonalisation_and_muon_training():
    G = torch.randn(48, 96)
    for coeffs, lo, hi in ((None, 0.6, 1.2), (POLAR_EXPRESS, 0.99, 1.01)):
        O = orthogonalize(G) if coeffs is None else orthogonalize(G, coeffs)
        s = torch.linalg.svdvals(O)
        assert lo < s.min() and s.max() < hi
        U, _, Vh = torch.linalg.svd(G, full_matrices=False)
        assert torch.allclose(O / s.mean(), (U @ Vh), atol=0.35)      # same singular vectors as G
    assert orthogonalize(G.t().contiguous()).shape == (96, 48)
    for name in ("muon", "normuon"):
        m = _model()
        cfg = PretrainingConfig(dataset_dir="x", optimizer=name, bf16=False)
        eng = MuonEngine(m, AdamWHyper(lr=1e-3), cfg, torch.device("cpu"))
        names = {s.name for s in eng.muon_slots}
        assert "model.layers.0.attn.Wqkv.weight" in names and "head.dense.weight" in names
        assert not any("tok_embeddings" in n or "norm" in n or "bias" in n for n in names)
        b = _batch()
        losses = []
        for _ in range(12):
            out = m(**b)
            out["loss"].backward()
            eng.step(1e-3, 1)
            losses.append(out["loss"].item())
        assert losses[-1] < losses[0] - 0.3, (name, losses)
