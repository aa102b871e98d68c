"""The encoder on the GPU kernels against the fp32 CPU restatement of the same model."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch(tok, n=24, width=256, rows=12, seed=1):
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    seqs = synthetic_token_sequences(n, 20, 200, seed=seed)
    coll = PackingCollator(tok, width, 0.3, target_rows=rows, batch_size=n, seed=seed)
    b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
    b.pop("num_real_tokens")
    return b


def test_encoder_loss_and_grads_match_cpu(cuda_status):
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine

    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=3, num_attention_heads=4,
                      max_position_embeddings=256)
    cpu = ProtEncoderMLM(cfg, tok)
    with torch.no_grad():  # output projections start at zero: give them values so every path matters
        for layer in cpu.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.03)
            layer.mlp.Wo.weight.normal_(0, 0.03)
    gpu = copy.deepcopy(cpu)
    engine = ShardedEngine(gpu, AdamWHyper(lr=1e-3), torch.device("cuda:0"))
    batch = _batch(tok)
    inputs = {k: batch[k] for k in ("input_ids", "cu_seqlens", "position_ids", "masked_idx", "masked_labels")}
    inputs["max_seqlen"] = batch["max_seqlen"]
    out_c = cpu(**inputs)
    out_c["loss"].backward()
    out_g = gpu(**{k: (v.cuda() if torch.is_tensor(v) else v) for k, v in inputs.items()})
    out_g["loss"].backward()
    engine.collect_autograd_grads()
    torch.cuda.synchronize()
    assert abs(out_c["loss"].item() - out_g["loss"].item()) < 3e-2, (out_c["loss"].item(), out_g["loss"].item())
    by_name = dict(cpu.named_parameters())
    worst = 0.0
    for s in engine.slots:
        g_ref = by_name[s.name].grad
        g = engine.main_grad[s.offset:s.offset + s.numel].view(s.shape).cpu()
        denom = g_ref.abs().max().item() + 1e-6
        rel = (g - g_ref).abs().max().item() / denom
        worst = max(worst, rel)
        assert rel < 0.08, f"{s.name}: rel err {rel:.4f} (max |g| {denom:.3e})"
    print("worst relative grad error", worst)


def test_training_reduces_loss_and_matches_cpu_trajectory(cuda_status):
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule

    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256)
    base = ProtEncoderMLM(cfg, tok)
    losses = {}
    for dev in ("cpu", "cuda:0"):
        m = copy.deepcopy(base)
        eng = ShardedEngine(m, AdamWHyper(lr=2e-3), torch.device(dev))
        m.train()
        st = TrainStep(m, eng, WarmupLinearSchedule(2e-3, 2, 1000), torch.device(dev))
        batches = [_batch(tok, seed=s) for s in range(3)]
        losses[dev] = [st.step_from_host([batches[i % 3]]) for i in range(12)]
    c, g = losses["cpu"], losses["cuda:0"]
    assert g[-1] < g[0] - 0.1, g
    for a, b in zip(c, g):
        assert abs(a - b) < 0.08, (c, g)


def test_checkpoint_roundtrip_gpu(tmp_path, cuda_status):
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule

    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                      max_position_embeddings=256)
    dev = torch.device("cuda:0")
    m = ProtEncoderMLM(cfg, tok)
    eng = ShardedEngine(m, AdamWHyper(lr=1e-3), dev)
    sch = WarmupLinearSchedule(1e-3, 2, 100)
    st = TrainStep(m, eng, sch, dev)
    b = _batch(tok)
    for _ in range(3):
        st.step_from_host([b])
    ckpt.save_checkpoint(eng, sch, 3, 0, str(tmp_path), 1, 10, 10)
    ref_next = st.step_from_host([b])
    m2 = ProtEncoderMLM(cfg, tok)
    eng2 = ShardedEngine(m2, AdamWHyper(lr=1e-3), dev)
    sch2 = WarmupLinearSchedule(1e-3, 2, 100)
    step, _ = ckpt.load_checkpoint(eng2, sch2, str(tmp_path / "checkpoint-3"))
    assert step == 3 and eng2.step_count == 3
    nxt = TrainStep(m2, eng2, sch2, dev).step_from_host([b])
    assert abs(nxt - ref_next) < 2e-3, (nxt, ref_next)
    sd = torch.load(tmp_path / "checkpoint-3" / "pytorch_model.bin")
    assert "decoder.weight" in sd and "model.layers.1.mlp.Wi.weight" in sd
    assert sd["model.layers.1.mlp.Wi.weight"].dtype == torch.float32


def test_padding_tail_trim_leaves_loss_and_grads_unchanged(cuda_status):
    """Cutting the padding tail off a static flat batch (host-known real-token count) must not
    change the loss or any gradient: the tail carries no label and attends to nothing real."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256)
    model = ProtEncoderMLM(cfg, tok)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.03)
            layer.mlp.Wo.weight.normal_(0, 0.03)
    engine = ShardedEngine(model, AdamWHyper(lr=1e-3), torch.device("cuda:0"))
    seqs = synthetic_token_sequences(16, 20, 120, seed=5)
    coll = PackingCollator(tok, 256, 0.3, target_rows=12, batch_size=16, seed=5)     # 3072 slots, ~1100 real
    b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
    n_real = int(b["num_real_tokens"])
    assert n_real + 256 < b["input_ids"].numel()
    keys = ("input_ids", "cu_seqlens", "position_ids", "masked_idx", "masked_labels", "max_seqlen")
    inputs = {k: (b[k].cuda() if torch.is_tensor(b[k]) else b[k]) for k in keys}
    grads, losses = [], []
    for trim in (None, n_real):
        engine.zero_grad()
        out = model(**inputs, num_real_tokens=trim)
        out["loss"].backward()
        engine.collect_autograd_grads()
        torch.cuda.synchronize()
        losses.append(out["loss"].item())
        grads.append(engine.main_grad.clone())
    assert abs(losses[0] - losses[1]) < 1e-5, losses
    scale = grads[0].abs().max().item()
    # weight gradients are fp32 atomic sums, so only the summation order may differ
    assert (grads[0] - grads[1]).abs().max().item() < 2e-3 * scale


@pytest.mark.parametrize("shape", [(4, 256, 512), (3, 512, 256), (2, 1024, 2048)])
def test_newton_schulz_on_grouped_gemm_matches_fp32(shape, cuda_status):
    """All matrices of a stack are orthogonalised by three row-grouped tcgen05 GEMM launches per
    iteration; the fp32 restatement runs the same iterations with torch.bmm on the CPU."""
    from nanoplm_b200.parallel import muon
    torch.manual_seed(3)
    G = torch.randn(*shape) * torch.tensor([0.1, 1.0, 7.0, 30.0])[:shape[0], None, None]   # norms differ
    ref = muon.orthogonalize_batched(G, muon.POLAR_EXPRESS)
    X = G.cuda().to(torch.bfloat16)
    assert muon._grouped_ok(X if shape[1] <= shape[2] else X.transpose(1, 2).contiguous())
    from nanoplm_b200.ops import _lib
    n0 = _lib.launches()
    out = muon.orthogonalize_batched(G.cuda(), muon.POLAR_EXPRESS).float().cpu()
    assert _lib.launches() - n0 == 3 * len(muon.POLAR_EXPRESS)
    assert out.shape == ref.shape
    for o, r in zip(out, ref):
        assert (o - r).norm().item() < 0.06 * r.norm().item(), ((o - r).norm().item(), r.norm().item())
        sv = torch.linalg.svdvals(o)
        assert 0.9 < sv.min().item() and sv.max().item() < 1.1


@pytest.mark.parametrize("optimizer", ["muon", "normuon"])
def test_muon_engine_trains_on_gpu_like_cpu(optimizer, cuda_status):
    from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper
    from nanoplm_b200.parallel.muon import MuonEngine
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule

    torch.manual_seed(0)
    tok = ProtTokenizer()
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256)
    base = ProtEncoderMLM(cfg, tok)
    losses = {}
    for dev in ("cpu", "cuda:0"):
        m = copy.deepcopy(base)
        pc = PretrainingConfig(dataset_dir="x", optimizer=optimizer, bf16=dev != "cpu", muon_learning_rate=5e-3)
        eng = MuonEngine(m, AdamWHyper(lr=1e-3), pc, torch.device(dev))
        m.train()
        st = TrainStep(m, eng, WarmupLinearSchedule(1e-3, 2, 1000), torch.device(dev))
        batches = [_batch(tok, seed=s) for s in range(3)]
        losses[dev] = [st.step_from_host([batches[i % 3]]) for i in range(10)]
    c, g = losses["cpu"], losses["cuda:0"]
    assert g[-1] < g[0] - 0.1, g
    for a, b in zip(c, g):
        assert abs(a - b) < 0.12, (c, g)


def test_fp32_compute_copy_on_the_gpu_follows_the_cpu_engine(cuda_status):
    """`bf16: false` on a GPU: the compute copy stays fp32, the optimizer kernels (which write a bf16
    copy) are not used, and training follows the CPU engine step by step; the same for the one-group
    optimizer of the distillation pipeline (`decay_all`)."""
    from nanoplm_b200.config.schema import ModelConfig, StudentConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.models.student import ProtX
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    s = ProtX(StudentConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2))
    c = copy.deepcopy(s)
    hyper = AdamWHyper(lr=1e-3, weight_decay=0.01)
    eg = ShardedEngine(s, hyper, dev, compute_dtype=torch.float32, decay_all=True)
    ec = ShardedEngine(c, hyper, torch.device("cpu"), compute_dtype=torch.float32, decay_all=True)
    assert not eg.kernel_opt and len(eg.optimizer_state_dict()["param_groups"]) == 1
    g = torch.Generator().manual_seed(1)
    for _ in range(3):
        grad = torch.randn(ec.total, generator=g) * 0.01
        ec.main_grad.copy_(grad)
        eg.main_grad.copy_(grad.cuda())
        a, b = float(ec.step(1e-3, 1)), float(eg.step(1e-3, 1))
        assert abs(a - b) < 1e-4 * a
    assert max(float((x.detach().cpu() - y.detach()).abs().max()) for x, y in zip(s.parameters(), c.parameters())) < 1e-5

    m = ProtEncoderMLM(ModelConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                                   max_position_embeddings=128), ProtTokenizer())
    with torch.no_grad():
        for layer in m.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            layer.mlp.Wo.weight.normal_(0, 0.05)
    mc = copy.deepcopy(m)
    hyper = AdamWHyper(lr=2e-3, weight_decay=0.05)
    eg = ShardedEngine(m, hyper, dev, compute_dtype=torch.float32)
    ec = ShardedEngine(mc, hyper, torch.device("cpu"), compute_dtype=torch.float32)
    ids = torch.randint(4, 24, (150,))
    cu = torch.tensor([0, 40, 90, 150], dtype=torch.int32)
    lab = torch.full((150,), -100)
    lab[::4] = ids[::4]
    for _ in range(3):
        lc = mc(input_ids=ids, labels=lab, cu_seqlens=cu)["loss"]
        lc.backward()
        lg = m(input_ids=ids.cuda(), labels=lab.cuda(), cu_seqlens=cu.cuda())["loss"]
        lg.backward()
        a, b = float(ec.step(2e-3, 1)), float(eg.step(2e-3, 1))
        assert abs(float(lc.detach()) - float(lg.detach())) < 2e-3 and abs(a - b) < 2e-2 * a
