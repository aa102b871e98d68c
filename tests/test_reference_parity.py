"""Parity with the reference implementation itself (the `nanoplm` package installed under
`baseline/_ref`, imported unmodified; every test here is skipped when it is absent).

  * same state dict -> same logits and loss in fp32 on padded input (the reference's SDPA route,
    modeling.py:631-752), and the same loss through this package's dynamic-packed and static-packed
    routes on the same sequences;
  * `pytorch_model.bin` / `optimizer.pt` written by one side load in the other
    (pure_pipeline.py:224-331);
  * tokenizer ids (tokenizer.py:20-62) including lower case and the U / Z / O / B residues;
  * packing-collator layout: cu_seqlens, position ids, flat length, padding sequences, and the MLM
    invariants of tests/test_packing_collator.py:57-255 checked on both collators;
  * the ProtX student (distillation/models/student/model.py:50-112): same keys, same raw and projected
    embeddings with the reference's weights, same tokenizer ids, same masked-MSE loss as the reference's
    distillation trainer (distillation/trainer.py:30-40);
  * batch arithmetic, worker count and run planning (pretraining/utils.py:28-265) for new and resumed runs;
  * shards written here are read by the reference's `ShardedDataset`, `.data_manifest` files go both ways;
  * the YAML templates the reference's `get-yaml` commands write load here with the reference's values, and its
    `params.yaml` drives this package's data pipeline to a dataset the reference's validators accept;
  * schedules, weight-decay and Muon routing, the FLOP estimate and the Polar-Express iteration;
  * the padded MLM collator, the shard validators, the initialisation, every command / option / default of
    the CLI, and ten optimizer steps of the reference's recipe step by step (pretraining and distillation);
  * one run directory handed from the reference's `run_pure_pretraining` to this package's `run_pretraining`
    and back, each resuming the other's checkpoint.
"""
import os
import sys
import types
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"

pytestmark = pytest.mark.skipif(not (REF / "nanoplm").exists(), reason="reference package not installed")


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    """The reference's modules, imported from baseline/_ref (it opens a log file under the current
    directory on import, hence the temporary cwd; optional third-party modules it imports without
    using on these paths get empty placeholders)."""
    work = tmp_path_factory.mktemp("refcwd")
    cwd = os.getcwd()
    os.chdir(work)
    added = []
    for name, attrs in (("IPython", {"get_ipython": lambda: None}), ("h5py", {"File": object}), ("Bio", {}),
                        ("Bio.SeqIO", {})):
        try:
            __import__(name)
        except Exception:
            m = types.ModuleType(name)
            for k, v in attrs.items():
                setattr(m, k, v)
            sys.modules[name] = m
            added.append(name)
    if "Bio" in added:
        sys.modules["Bio"].SeqIO = sys.modules["Bio.SeqIO"]
    sys.path.insert(0, str(REF))
    try:
        from nanoplm.pretraining import collator as ref_collator
        from nanoplm.pretraining import pure_pipeline as ref_pipeline
        from nanoplm.pretraining.models.modern_bert.model import ProtModernBertMLMConfig
        from nanoplm.pretraining.models.modern_bert.pure_model import PureProtModernBertMLM
        from nanoplm.pretraining.models.modern_bert.tokenizer import ProtModernBertTokenizer
    except Exception as exc:  # pragma: no cover
        os.chdir(cwd)
        pytest.skip(f"reference import failed: {type(exc).__name__}: {exc}")
    ns = types.SimpleNamespace(collator=ref_collator, pipeline=ref_pipeline, Config=ProtModernBertMLMConfig,
                               Model=PureProtModernBertMLM, Tokenizer=ProtModernBertTokenizer)
    yield ns
    os.chdir(cwd)
    sys.path.remove(str(REF))
    for name in added:
        sys.modules.pop(name, None)


GEOM = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=2,
            max_position_embeddings=256)


def _pair(ref):
    """(reference model, this package's model) with the reference's weights copied across."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    rm = ref.Model(ref.Config(vocab_size=32, **GEOM)).float().eval()
    with torch.no_grad():   # the reference zero-initialises some projections; make every path matter
        for p in rm.parameters():
            if p.ndim >= 2:
                p.add_(torch.randn_like(p) * 0.05)
    om = ProtEncoderMLM(ModelConfig(**GEOM), ProtTokenizer()).float().eval()
    missing, unexpected = om.load_state_dict(rm.state_dict(), strict=True), None
    return rm, om


def _sequences(n, lo, hi, seed):
    from nanoplm_b200.data.synthetic import synthetic_sequences
    return synthetic_sequences(n, lo, hi, seed)


def test_state_dict_keys_and_shapes_are_identical(ref):
    rm, om = _pair(ref)
    a, b = rm.state_dict(), om.state_dict()
    assert list(a.keys()) == list(b.keys())
    assert all(a[k].shape == b[k].shape for k in a)
    assert sum(p.numel() for p in rm.parameters()) == sum(p.numel() for p in om.parameters())


def test_same_weights_give_same_logits_and_loss_on_padded_input(ref):
    rm, om = _pair(ref)
    tok = ref.Tokenizer()
    seqs = _sequences(6, 5, 90, seed=3)
    enc = tok(seqs, padding=True, return_tensors="pt")
    ids, mask = enc["input_ids"], enc["attention_mask"]
    labels = torch.full_like(ids, -100)
    g = torch.Generator().manual_seed(1)
    pick = (torch.rand(ids.shape, generator=g) < 0.3) & mask.bool()
    labels[pick] = ids[pick]
    with torch.no_grad():
        r = rm(input_ids=ids, attention_mask=mask, labels=labels)
        o = om(input_ids=ids, attention_mask=mask, labels=labels)
        r_logits = rm(input_ids=ids, attention_mask=mask)["logits"]
        o_logits = om(input_ids=ids, attention_mask=mask)["logits"]
    assert abs(float(r["loss"]) - float(o["loss"])) < 2e-5
    real = mask.bool()
    assert (r_logits[real] - o_logits[real]).abs().max().item() < 2e-4


def test_packed_routes_reproduce_the_reference_loss(ref):
    """Dynamic (2-D rows + cu_seqlens) and static (flat, fixed length) packed batches of the same
    sequences and the same labels give the loss the reference computes on the padded batch."""
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    rm, om = _pair(ref)
    tok = ProtTokenizer()
    seqs = _sequences(10, 5, 60, seed=9)
    examples = [{"input_ids": torch.tensor(tok.encode(s))} for s in seqs]
    for static in (False, True):
        coll = PackingCollator(tok, 64, 0.3, target_rows=8 if static else None,
                               batch_size=len(examples) if static else None, seed=4)
        b = coll(examples)
        b.pop("num_real_tokens", None)
        with torch.no_grad():
            o = om(**{k: v for k, v in b.items() if k in ("input_ids", "attention_mask", "labels", "cu_seqlens",
                                                          "max_seqlen", "position_ids")})
        # rebuild the padded view of the very same (masked) tokens and labels, sequence by sequence
        flat_ids = b["input_ids"].reshape(-1)
        flat_lab = b["labels"].reshape(-1)
        if not static:
            keep = b["attention_mask"].reshape(-1).bool()
            flat_ids, flat_lab = flat_ids[keep], flat_lab[keep]
        cu = b["cu_seqlens"].tolist()
        rows = [(flat_ids[s:e], flat_lab[s:e]) for s, e in zip(cu[:-1], cu[1:]) if e > s and flat_ids[s] != tok.pad_token_id]
        L = max(len(r[0]) for r in rows)
        ids = torch.full((len(rows), L), tok.pad_token_id, dtype=torch.long)
        lab = torch.full((len(rows), L), -100, dtype=torch.long)
        msk = torch.zeros((len(rows), L), dtype=torch.long)
        for i, (a, l) in enumerate(rows):
            ids[i, :len(a)], lab[i, :len(a)], msk[i, :len(a)] = a, l, 1
        with torch.no_grad():
            r = rm(input_ids=ids, attention_mask=msk, labels=lab)
        assert abs(float(r["loss"]) - float(o["loss"])) < 3e-5, f"static={static}"


def test_checkpoints_are_interchangeable(ref, tmp_path):
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    rm, om = _pair(ref)
    om.train()
    hyper = AdamWHyper(lr=1e-3, weight_decay=0.01)
    eng = ShardedEngine(om, hyper, torch.device("cpu"))
    tok = ref.Tokenizer()
    enc = tok(_sequences(4, 10, 40, seed=5), padding=True, return_tensors="pt")
    labels = enc["input_ids"].clone()
    labels[enc["attention_mask"] == 0] = -100
    for _ in range(2):
        om(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)["loss"].backward()
        eng.step(1e-3, 1)
    sched = WarmupLinearSchedule(1e-3, 1, 10)
    d = ckpt.save_checkpoint(eng, sched, 2, 0, str(tmp_path), 1, 1, 1)
    # (a) this package's files load through the reference's own loader into its model + AdamW
    cfg = types.SimpleNamespace(optimizer="adamw", adam_weight_decay=0.01, adam_learning_rate=1e-3,
                                adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8)
    r2 = ref.Model(ref.Config(vocab_size=32, **GEOM)).float()
    opt = ref.pipeline._create_optimizer(r2, cfg)
    lam = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0)
    torch.save(lam.state_dict(), Path(d) / "scheduler.pt")   # the reference's scheduler is a LambdaLR
    step, epoch = ref.pipeline._load_checkpoint(r2, opt, lam, str(d), torch.device("cpu"))
    assert (step, epoch) == (2, 0)
    full = eng.full_state_dict_model()
    for k, v in r2.state_dict().items():
        assert torch.equal(v, full[k]), k
    st = opt.state_dict()["state"]
    assert len(st) == len(list(r2.parameters())) and all(float(s["step"]) == 2.0 for s in st.values())
    named = dict(r2.named_parameters())
    decay = [n for n, p in named.items() if ref.pipeline._use_weight_decay(n, p)]
    first = opt.state[named[decay[0]]]["exp_avg"]
    assert first.shape == named[decay[0]].shape and first.abs().sum() > 0
    # (b) files written by the reference's saver load here
    out = tmp_path / "refrun"
    ref.pipeline._save_checkpoint(r2, opt, lam, 7, 1, str(out), 1, 1, 1)
    om2 = type(om)(om.config, om.tokenizer).float()
    eng2 = ShardedEngine(om2, hyper, torch.device("cpu"))
    sched2 = WarmupLinearSchedule(1e-3, 1, 10)
    torch.save(sched.state_dict(), out / "checkpoint-7" / "scheduler.pt")
    step, epoch = ckpt.load_checkpoint(eng2, sched2, str(out / "checkpoint-7"))
    assert (step, epoch) == (7, 1)
    back = eng2.full_state_dict_model()
    for k, v in r2.state_dict().items():
        assert torch.equal(v, back[k]), k
    a, b = eng.optimizer_state_dict()["state"], eng2.optimizer_state_dict()["state"]
    assert a.keys() == b.keys() and all(torch.equal(a[i]["exp_avg_sq"], b[i]["exp_avg_sq"]) for i in a)


def test_tokenizer_ids_match(ref):
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    rt, ot = ref.Tokenizer(), ProtTokenizer()
    seqs = ["MKTAYIAKQR", "mktayiakqr", "ACDEFGHIKLMNPQRSTVWY", "UZOBXuzobx", "A", "MKT" * 50]
    assert rt.get_vocab() == ot.get_vocab()
    for name in ("pad_token_id", "eos_token_id", "unk_token_id", "mask_token_id"):
        assert getattr(rt, name) == getattr(ot, name), name
    assert sorted(rt.all_special_ids) == sorted(ot.all_special_ids)
    for s in seqs:
        assert rt.encode(s) == ot.encode(s), s
    a = rt(seqs, padding=True, return_tensors="pt")
    b = ot(seqs, padding=True, return_tensors="pt")
    assert torch.equal(a["input_ids"], b["input_ids"]) and torch.equal(a["attention_mask"], b["attention_mask"])
    a = rt(seqs, padding="max_length", max_length=32, truncation=True, return_tensors="pt")
    b = ot(seqs, padding="max_length", max_length=32, truncation=True, return_tensors="pt")
    assert torch.equal(a["input_ids"], b["input_ids"])


@pytest.mark.parametrize("static", [False, True], ids=["dynamic", "static"])
def test_packing_collator_layout_matches(ref, static):
    """Both collators pack first-fit-decreasing: with masking off they must emit the same tokens,
    cu_seqlens and position ids; with masking on, the invariants of the reference's own collator
    tests hold for both."""
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    rt, ot = ref.Tokenizer(), ProtTokenizer()
    seqs = _sequences(12, 3, 60, seed=21)
    ex_r = [{"input_ids": torch.tensor(rt.encode(s))} for s in seqs]
    ex_o = [{"input_ids": torch.tensor(ot.encode(s))} for s in seqs]
    kw = dict(target_rows=8, batch_size=len(seqs)) if static else {}
    rc = ref.collator.PackingCollator(rt, 64, mlm_probability=0.0, **kw)
    oc = PackingCollator(ot, 64, 0.0, seed=0, **kw)
    a, b = rc(ex_r), oc(ex_o)
    assert torch.equal(a["input_ids"], b["input_ids"])
    assert torch.equal(a["cu_seqlens"].to(torch.int32), b["cu_seqlens"].to(torch.int32))
    assert int(a["max_seqlen"]) == int(b["max_seqlen"])
    if static:
        assert torch.equal(a["position_ids"], b["position_ids"])
        assert a["input_ids"].shape == (8 * 64,) and a["cu_seqlens"].numel() == len(seqs) + 1 + 8
    else:
        assert torch.equal(a["attention_mask"], b["attention_mask"])
    assert bool((a["labels"] == -100).all()) and bool((b["labels"] == -100).all())
    # masking on: invariants (labels only on real non-special tokens, the original id as label,
    # replaced ids inside the amino-acid pool, roughly the requested fraction)
    rc = ref.collator.PackingCollator(rt, 64, mlm_probability=0.3, **kw)
    oc = PackingCollator(ot, 64, 0.3, seed=1, **kw)
    clean = a["input_ids"].reshape(-1)
    special = torch.tensor(sorted(ot.all_special_ids))
    for out in (rc(ex_r), oc(ex_o)):
        ids, lab = out["input_ids"].reshape(-1), out["labels"].reshape(-1)
        m = lab != -100
        assert torch.equal(lab[m], clean[m])
        assert not torch.isin(clean[m], special).any()
        assert torch.equal(ids[~m], clean[~m])
        changed = ids[m] != clean[m]
        pool_or_mask = (ids[m][changed] == ot.mask_token_id) | (ids[m][changed] >= 4)
        assert bool(pool_or_mask.all())
        n_real = int((~torch.isin(clean, special)).sum())
        assert 0.15 < m.sum().item() / n_real < 0.45


def test_dropout_settings_are_honoured_or_refused(ref):
    """mlp_dropout changes the training forward (and only that); a non-zero attention_dropout,
    which the attention kernels cannot honour, is refused instead of being dropped silently."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    with pytest.raises(ValueError, match="attention_dropout"):
        ModelConfig(attention_dropout=0.1, **GEOM)
    tok = ProtTokenizer()
    torch.manual_seed(0)
    m = ProtEncoderMLM(ModelConfig(mlp_dropout=0.5, embedding_dropout=0.1, **GEOM), tok).float()
    with torch.no_grad():
        for layer in m.model.layers:
            layer.mlp.Wo.weight.normal_(0, 0.05)
    enc = tok(_sequences(3, 10, 40, seed=2), padding=True, return_tensors="pt")
    labels = enc["input_ids"].clone()
    labels[enc["attention_mask"] == 0] = -100
    kw = dict(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)
    m.eval()
    with torch.no_grad():
        e1, e2 = float(m(**kw)["loss"]), float(m(**kw)["loss"])
    assert e1 == e2                                   # no dropout in eval mode
    m.train()
    with torch.no_grad():
        t1, t2 = float(m(**kw)["loss"]), float(m(**kw)["loss"])
    assert t1 != t2 and abs(t1 - e1) > 1e-6           # active, and random, in training mode


def test_hf_trainer_checkpoint_layout_resumes_here(ref, tmp_path):
    """`checkpoint-N/{model.safetensors, optimizer.pt, scheduler.pt, trainer_state.json}` as the
    reference's HF-Trainer pipeline leaves it (pipeline.py:293-295) loads into this engine: weights
    (tied decoder stored once), AdamW moments in [decay | no-decay] order, step from trainer_state."""
    import json
    from safetensors.torch import save_file
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    rm, om = _pair(ref)
    rm.train()
    cfg = types.SimpleNamespace(optimizer="adamw", adam_weight_decay=0.01, adam_learning_rate=1e-3,
                                adam_beta1=0.9, adam_beta2=0.999, adam_epsilon=1e-8)
    opt = ref.pipeline._create_optimizer(rm, cfg)     # same grouping rule as the HF Trainer's
    tok = ref.Tokenizer()
    enc = tok(_sequences(4, 10, 40, seed=8), padding=True, return_tensors="pt")
    labels = enc["input_ids"].clone()
    labels[enc["attention_mask"] == 0] = -100
    rm(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)["loss"].backward()
    opt.step()
    d = tmp_path / "checkpoint-7"
    d.mkdir()
    sd = {k: v.detach().clone().contiguous() for k, v in rm.state_dict().items() if k != "decoder.weight"}
    save_file(sd, str(d / "model.safetensors"))
    torch.save(opt.state_dict(), d / "optimizer.pt")
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0)
    torch.save(sched.state_dict(), d / "scheduler.pt")
    (d / "trainer_state.json").write_text(json.dumps({"global_step": 7, "epoch": 1.25, "log_history": []}))
    eng = ShardedEngine(om, AdamWHyper(lr=1e-3, weight_decay=0.01), torch.device("cpu"))
    step, epoch = ckpt.load_checkpoint(eng, WarmupLinearSchedule(1e-3, 1, 10), str(d))
    assert (step, epoch) == (7, 1)
    full = eng.full_state_dict_model()
    for k, v in rm.state_dict().items():
        assert torch.allclose(full[k], v.detach(), atol=1e-7), k
    assert eng.step_count == 1
    named = [n for n, p in rm.named_parameters()]
    decay = [n for n, p in rm.named_parameters() if ref.pipeline._use_weight_decay(n, p)]
    mine = eng.optimizer_state_dict()["state"]
    theirs = opt.state_dict()["state"]
    assert len(mine) == len(theirs) == len(named)
    assert all(torch.allclose(mine[i]["exp_avg"], theirs[i]["exp_avg"], atol=1e-8) for i in theirs)
    assert len(decay) == len([s for s in eng.slots if s.decay])


def test_student_protx_matches_the_reference_student(ref):
    """The reference's ProtX (its SwiGLU ModernBERT body + 1024-wide projection + T5 norm,
    distillation/models/student/model.py:50-112) and this package's student share state-dict keys; with
    the reference's weights copied across they give the same raw and projected embeddings on a padded
    batch, the two tokenizers give the same ids, and the masked MSE of the distillation trainer
    (distillation/trainer.py:30-40) agrees with `ops.functional.masked_mse`."""
    try:
        from nanoplm.distillation.models.student.model import ProtX as RefProtX, ProtXConfig as RefCfg
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference student import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.config.schema import StudentConfig
    from nanoplm_b200.models.student import ProtX
    from nanoplm_b200.ops import functional as ops
    torch.manual_seed(0)
    geom = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=2)
    rm = RefProtX(RefCfg(**geom)).float().eval()
    with torch.no_grad():
        for p in rm.parameters():
            if p.ndim >= 2:
                p.add_(torch.randn_like(p) * 0.05)
    om = ProtX(StudentConfig(max_position_embeddings=8192, **geom)).float().eval()
    assert set(om.state_dict()) == set(rm.state_dict())
    om.load_state_dict(rm.state_dict(), strict=True)
    seqs = ["MKTAYIAKQRQISFVKSHFSRQ", "ACDEFGHIKLMNPQRSTVWY" * 8, "MK", "mktay" + "UZOB"]
    enc = rm.tokenizer(seqs, padding=True, return_tensors="pt")
    for s in seqs:
        assert om.tokenizer.encode(s) == rm.tokenizer(s)["input_ids"], s
    keep = enc["attention_mask"].bool()
    with torch.no_grad():
        for training_mode in (False, True):
            a = rm(enc["input_ids"], enc["attention_mask"], training_mode=training_mode).last_hidden_state
            b = om(enc["input_ids"], enc["attention_mask"], training_mode=training_mode)
            b = b["last_hidden_state"] if isinstance(b, dict) else b.last_hidden_state
            assert a.shape == b.shape
            assert (a[keep] - b[keep]).abs().max().item() < 2e-5 * max(1.0, a[keep].abs().max().item())
        # the trainer's loss: sum over features of the squared error, mean over real tokens
        teacher = torch.randn_like(a)
        m = enc["attention_mask"].unsqueeze(-1).to(a.dtype)
        ref_loss = (((a - teacher) ** 2) * m).sum() / m.sum().clamp(min=1.0)
        own = ops.masked_mse(b.reshape(-1, b.shape[-1]), teacher.reshape(-1, b.shape[-1]),
                             enc["attention_mask"].reshape(-1))
        assert abs(own.item() - ref_loss.item()) < 1e-3 * abs(ref_loss.item())


def test_batch_setup_worker_count_and_run_planning_match(ref, tmp_path, monkeypatch):
    """`compute_batch_setup`, `get_num_workers` and `prepare_run_and_steps` of the reference
    (pretraining/utils.py:28-265) against `runtime/run_dirs.py` on a grid of settings, for a new run
    and for a resume (run directory, W&B name with the resume counter, archived later checkpoints,
    epochs and clamped step intervals)."""
    try:
        from nanoplm.pretraining import utils as ref_utils
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference utils import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.runtime import run_dirs
    for gbs in (1, 4096, 2 ** 20, 3 * 10 ** 6):
        for mbs in (1, 8, 64):
            for seq in (64, 512, 1024):
                for world in (1, 2, 8):
                    cfg = types.SimpleNamespace(global_batch_size=gbs, micro_batch_size=mbs)
                    a = ref_utils.compute_batch_setup(cfg, seq, world)
                    b = run_dirs.compute_batch_setup(gbs, mbs, seq, world)
                    assert (a.grad_accum_steps, a.global_batch_size_samples, a.achieved_global_batch_tokens) == \
                           (b.grad_accum_steps, b.global_batch_size_samples, b.achieved_global_batch_tokens)
    for value in ("auto", 0, 3, "5"):
        for world in (1, 4, 8):
            assert ref_utils.get_num_workers(value, world) == run_dirs.get_num_workers(value, world)
    for bad in ("many", -1):
        with pytest.raises(ValueError):
            ref_utils.get_num_workers(bad, 1)
        with pytest.raises(ValueError):
            run_dirs.get_num_workers(bad, 1)

    def both(kind, resume, extra, epochs, log, ev, save, samples, batch):
        out = []
        for side in ("ref", "own"):
            root = tmp_path / f"{kind}-{side}"
            ck = root / "run-01010101" / "checkpoint-20"
            if resume:
                for step in (10, 20, 30, 40):
                    (root / "run-01010101" / f"checkpoint-{step}").mkdir(parents=True)
            if side == "ref":
                pc = types.SimpleNamespace(ckp_dir=str(root), num_epochs=epochs, logging_steps=log, eval_steps=ev,
                                           save_steps=save)
                rc = types.SimpleNamespace(is_resume=resume, checkpoint_dir=str(ck), extra_epochs=extra)
                name, wb, outdir, n_ep, ls, es, ss, rstep = ref_utils.prepare_run_and_steps(pc, rc, samples, batch)
            else:
                p = run_dirs.prepare_run_and_steps(str(root), epochs, log, ev, save, resume, str(ck), extra, samples,
                                                   batch)
                name, wb, outdir, n_ep, ls, es, ss, rstep = (p.run_name, p.wandb_run_name, p.output_dir, p.num_epochs,
                                                             p.logging_steps, p.eval_steps, p.save_steps, p.resume_step)
            rel = Path(outdir).relative_to(root)
            listing = sorted(str(q.relative_to(root / rel)).split("/")[0].split("_")[0] + ":" + q.name
                             for q in (root / rel).rglob("checkpoint-*"))
            out.append((name.startswith("run-"), wb.replace(name, "RUN"), n_ep, ls, es, ss, rstep, listing,
                        (root / rel / ".resume_counter").read_text() if resume else None))
        assert out[0] == out[1], (kind, out)
        return out[0]

    new = both("new", False, None, 3, 10, 5000, 7, 1000, 64)
    assert new[2:7] == (3, 10, 48, 7, None)                       # 16 steps per epoch, eval clamped to 48
    res = both("resume", True, 2, 3, 10, 25, 7, 1000, 64)
    assert res[1] == "RUN-re1" and res[2] == 5 and res[6] == 20
    assert [x for x in res[7] if x.startswith("archived")] == ["archived:checkpoint-30", "archived:checkpoint-40"]


def test_shards_and_manifests_are_read_by_the_reference_and_back(ref, tmp_path):
    """Shards written by this package's `ShardWriter` are read by the reference's `ShardedDataset`
    (pretraining/dataset.py:147-290) with identical examples; a `.data_manifest` written by either side is
    read by the other (data/manifest.py:129-226) with the same fields and dataset paths."""
    try:
        from nanoplm.data import manifest as ref_manifest
        from nanoplm.pretraining import dataset as ref_dataset
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference data modules import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.data import manifest as own_manifest
    from nanoplm_b200.data.shards import ShardedDataset, ShardWriter
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    write_synthetic_fasta(tmp_path / "x.fasta", 57, 5, 90, seed=3)
    ShardWriter(tmp_path / "x.fasta", ProtTokenizer(), 64, tmp_path / "train", samples_per_shard=20,
                max_workers=1).create_shards()
    theirs, ours = ref_dataset.ShardedDataset(str(tmp_path / "train")), ShardedDataset(str(tmp_path / "train"))
    assert len(theirs) == len(ours) == 57
    for i in range(57):
        a, b = theirs[i], ours[i]
        assert set(a) == set(b)
        for k in a:
            assert torch.equal(torch.as_tensor(a[k]), torch.as_tensor(b[k])), (i, k)
    fields = dict(pipeline_mode="pretrain", seqs_num=70, min_seq_len=5, max_seq_len=64, val_ratio=0.2,
                  train_dir="train", val_dir="val", train_sequences=57, val_sequences=13, sharded=True,
                  samples_per_shard=20)
    own_manifest.write_manifest(tmp_path / "a", own_manifest.PretrainManifest(**fields))
    ref_manifest.write_manifest(tmp_path / "b", ref_manifest.PretrainManifest(**fields))
    for d in ("a", "b"):
        x, y = ref_manifest.read_manifest(tmp_path / d), own_manifest.read_manifest(tmp_path / d)
        for k in fields:
            assert getattr(x, k) == getattr(y, k) == fields[k], (d, k)
        ref_manifest.validate_manifest_for_pipeline(x, "pretrain")
        own_manifest.validate_manifest_for_pipeline(y, "pretrain")
        theirs_p, ours_p = ref_manifest.get_dataset_paths(tmp_path / d, x), own_manifest.get_dataset_paths(tmp_path / d, y)
        assert {k: str(v) for k, v in theirs_p.items()} == {k: str(v) for k, v in ours_p.items()}


def _ref_cli_modules():
    """The reference's cli sub-modules (the names `pretrain`, `distill`, `data` in `nanoplm.cli` are
    click groups that shadow the modules, hence the look-up through sys.modules)."""
    try:
        from nanoplm.cli import cli as ref_cli
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference cli import failed: {type(exc).__name__}: {exc}")
    return ref_cli, sys.modules["nanoplm.cli.pretrain"], sys.modules["nanoplm.cli.distill"]


def test_reference_yaml_templates_load_here_with_the_reference_values(ref, tmp_path, monkeypatch):
    """The templates written by the reference's own `get-yaml` commands (cli/pretrain.py:594-695,
    cli/distill.py:540-619) are the schema contract: this package's loaders accept them unchanged and
    give, field by field, what the reference's loaders give (cli/pretrain.py:704-924,
    cli/distill.py:629-743)."""
    import dataclasses

    import yaml
    from click.testing import CliRunner

    from nanoplm_b200.config import loaders
    ref_cli, ref_pre, ref_dis = _ref_cli_modules()
    monkeypatch.chdir(tmp_path)
    runner = CliRunner()
    assert runner.invoke(ref_cli, ["pretrain", "get-yaml", "pretrain.yaml"]).exit_code == 0
    assert runner.invoke(ref_cli, ["distill", "get-yaml", "distill.yaml"]).exit_code == 0

    raw = yaml.safe_load((tmp_path / "pretrain.yaml").read_text())
    pairs = [(ref_pre._load_model_config(raw["model"]), loaders.load_model_config(raw["model"]), ()),
             (ref_pre._load_pretrain_config(raw["pretraining"]), loaders.load_pretrain_config(raw["pretraining"]), ()),
             (ref_pre._load_resume_config(raw["resume"]), loaders.load_resume_config(raw["resume"]), ())]
    theirs_on, theirs_pt = ref_pre._resolve_pure_torch_config(raw["pure_torch"])
    ours_on, ours_pt = loaders.resolve_pure_torch_config(raw["pure_torch"])
    assert theirs_on == ours_on
    pairs.append((theirs_pt, ours_pt, ()))

    raw = yaml.safe_load((tmp_path / "distill.yaml").read_text())
    # `sharded: None` means "take it from the manifest" there; here the manifest always decides
    pairs += [(ref_dis._load_model_config(raw["model"]), loaders.load_student_config(raw["model"]), ()),
              (ref_dis._load_distill_config(raw["distillation"]), loaders.load_distill_config(raw["distillation"]),
               ("sharded",)),
              (ref_dis._load_resume_config(raw["resume"]), loaders.load_resume_config(raw["resume"]), ())]
    checked = 0
    for theirs, ours, skip in pairs:
        for k, v in dataclasses.asdict(theirs).items():
            if k in skip:
                continue
            assert hasattr(ours, k), (type(theirs).__name__, k)
            assert getattr(ours, k) == v, (type(theirs).__name__, k, v, getattr(ours, k))
            checked += 1
    assert checked > 90

    # the error contract of the loaders: same refusals on both sides
    pre = yaml.safe_load((tmp_path / "pretrain.yaml").read_text())
    import click
    for mutate in (lambda d: d["pretraining"].update(gradient_accumulation_steps=2),
                   lambda d: d["pretraining"].pop("dataset_dir"),
                   lambda d: d["pretraining"].update(no_such_key=1),
                   lambda d: d["model"].update(no_such_key=1),
                   lambda d: d["model"].pop("vocab_size")):
        bad = {k: dict(v) for k, v in pre.items()}
        mutate(bad)
        with pytest.raises((click.ClickException, ValueError)):
            ref_pre._load_model_config(bad["model"])
            ref_pre._load_pretrain_config(bad["pretraining"])
        with pytest.raises(loaders.ConfigError):
            loaders.load_model_config(bad["model"])
            loaders.load_pretrain_config(bad["pretraining"])


def test_reference_params_template_drives_the_data_pipeline_here(ref, tmp_path, monkeypatch):
    """`params.yaml` as written by the reference's `data get-yaml` (cli/data.py:676-725), pointed at a
    local FASTA, runs through this package's `data from-yaml`; the reference's validators then accept
    the result (data/validation.py:182-354, data/manifest.py:181-274)."""
    import yaml
    from click.testing import CliRunner

    from nanoplm_b200.cli import cli as own_cli
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    ref_cli, _, _ = _ref_cli_modules()
    try:
        from nanoplm.data import manifest as ref_manifest
        from nanoplm.data import validation as ref_validation
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference data modules import failed: {type(exc).__name__}: {exc}")
    monkeypatch.chdir(tmp_path)
    runner = CliRunner()
    assert runner.invoke(ref_cli, ["data", "get-yaml", str(tmp_path)]).exit_code == 0
    params = yaml.safe_load((tmp_path / "params.yaml").read_text())
    params["data_params"].update(seqs_num=60, min_seq_len=10, max_seq_len=64, val_ratio=0.2)
    params["pretrain_config"].update(samples_per_shard=20, max_workers=1)
    params["data_dirs"].update(url="unused", compressed_fasta="raw/x.fasta.gz", extracted_fasta="raw/x.fasta",
                               shuffled_fasta="raw/x_shuf.fasta", filtered_fasta="raw/x_filt.fasta",
                               splitted_fasta_dir="raw/split")
    (tmp_path / "params.yaml").write_text(yaml.safe_dump(params))
    write_synthetic_fasta(tmp_path / "raw" / "x.fasta", 120, 5, 80, seed=11)
    r = runner.invoke(own_cli, ["data", "from-yaml", "params.yaml", "--runner", "builtin"])
    assert r.exit_code == 0, r.output + str(r.exception)
    out = tmp_path / params["pretrain_config"]["output_dir"]
    m = ref_manifest.read_manifest(out)
    ref_manifest.validate_manifest_for_pipeline(m, "pretrain")
    assert (m.train_sequences, m.val_sequences, m.max_seq_len, m.samples_per_shard) == (48, 12, 64, 20)
    paths = ref_manifest.get_dataset_paths(out, m)
    res = ref_validation.validate_pretrain_dataset(out)
    assert len(res["train_shards"]) == 3 and len(res["val_shards"]) == 1
    assert Path(paths["train_dir"]).is_dir() and Path(paths["val_dir"]).is_dir()


def test_schedules_parameter_routing_flops_and_polar_express_match(ref):
    """The small rules of the training recipe, evaluated by the reference's own functions and by this
    package's: the warm-up / linear-decay schedule (pure_pipeline.py:150-172) step by step, the four
    distillation schedules (distillation/pipeline.py:396-446), weight-decay routing
    (pure_pipeline.py:68-76), Muon / AdamW routing (optim.py:19-60, 187-205), the FLOP estimate
    (pure_pipeline.py:86-104) and the Polar-Express orthogonalisation (optim.py:85-118)."""
    import math

    from nanoplm_b200.models.encoder import estimate_flops_per_token
    from nanoplm_b200.parallel import muon
    from nanoplm_b200.parallel.engine import use_weight_decay
    from nanoplm_b200.runtime import schedule
    P = ref.pipeline
    # pretraining schedule
    for total, ratio in ((100, 0.05), (37, 0.1), (10, 3), (1, 0.5), (50, 0.0)):
        w = P._get_warmup_steps(total, ratio)
        assert w == schedule.get_warmup_steps(total, ratio)
        opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.25)
        theirs = P._create_scheduler(opt, w, total)
        ours = schedule.WarmupLinearSchedule(0.25, w, total)
        for _ in range(total + 2):
            assert math.isclose(theirs.get_last_lr()[0], ours.get_last_lr()[0], rel_tol=1e-12, abs_tol=1e-15)
            opt.step(); theirs.step(); ours.step()
        sd = theirs.state_dict()
        again = schedule.WarmupLinearSchedule(0.25, w, total)
        again.load_state_dict(sd)
        assert again.last_epoch == sd["last_epoch"] and math.isclose(again.get_last_lr()[0], theirs.get_last_lr()[0],
                                                                      abs_tol=1e-15)
    for n, accum in ((0, 4), (1, 4), (8, 4), (9, 4), (9, 1)):
        assert P._num_update_steps_per_epoch(n, accum) == schedule.num_update_steps_per_epoch(n, accum)

    # distillation schedules; an explicit num_warmup_steps among the arguments wins on both sides
    D = sys.modules.get("nanoplm.distillation.pipeline")
    if D is None:
        import importlib
        D = importlib.import_module("nanoplm.distillation.pipeline")
    for name in ("cosine", "linear", "polynomial", "constant"):
        for kwargs in ({}, {"num_warmup_steps": 7}):
            total = 60
            opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1e-3)
            theirs = D._get_scheduler(opt, name, dict(kwargs), total)
            default_warmup = 0 if name == "constant" else int(total * 0.05)
            ours = schedule.make_distill_schedule(name, 1e-3, default_warmup, total, **kwargs)
            for _ in range(total + 1):
                assert math.isclose(theirs.get_last_lr()[0], ours.get_last_lr()[0], rel_tol=1e-9, abs_tol=1e-15), name
                opt.step(); theirs.step(); ours.step()
    with pytest.raises(ValueError):
        D._get_scheduler(opt, "nope", {}, 10)
    with pytest.raises(ValueError):
        schedule.make_distill_schedule("nope", 1e-3, 0, 10)

    # routing on the reference's own model
    rm, om = _pair(ref)
    O = sys.modules["nanoplm.pretraining.optim"]
    for name, p in rm.named_parameters():
        assert P._use_weight_decay(name, p) == use_weight_decay(name, p), name
        to_muon = p.ndim == 2 and not O._is_embedding_or_unembedding_param(name)
        ours_muon = p.ndim == 2 and not muon.is_embedding_or_unembedding(name)
        assert to_muon == ours_muon, name
    for name in ("lm_head.weight", "x.Embedding.weight", "decoder.bias", "a.unembedding", "layers.0.mlp.Wi.weight"):
        assert O._is_embedding_or_unembedding_param(name) == muon.is_embedding_or_unembedding(name), name

    cfg = om.config
    for s in (64, 512, 1024):
        assert P._estimate_model_flops_per_token(cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, s,
                                                 cfg.vocab_size) == estimate_flops_per_token(cfg, s)

    # Polar Express: same coefficients, and the same polar factor as the reference's (bf16) iteration
    assert len(O.polar_express_coeffs) == len(muon.POLAR_EXPRESS)
    for x, y in zip(O.polar_express_coeffs, muon.POLAR_EXPRESS):
        assert all(math.isclose(a, b, rel_tol=1e-15) for a, b in zip(x, y))
    plain = getattr(O._polar_express_paper, "_torchdynamo_orig_callable", None) or getattr(
        O._polar_express_paper, "__wrapped__", None)
    if plain is not None:                       # the undecorated function: no compiler run on the CPU
        torch.manual_seed(0)
        for shape in ((48, 96), (96, 48), (64, 64)):
            G = torch.randn(*shape)
            theirs = plain(G).float()
            ours = muon.orthogonalize(G, muon.POLAR_EXPRESS).float()
            assert ours.shape == theirs.shape
            # the reference iterates in bf16, this package in fp32 on the CPU: compare as polar factors
            assert (ours - theirs).norm() / theirs.norm() < 0.03
            s = torch.linalg.svdvals(ours)
            assert s.max() < 1.2 and s.min() > 0.5


def test_padding_collator_matches_the_reference_collator(ref):
    """The padded MLM collator (pretraining/collator.py:7-147): with masking off both give the same
    padded batch; with masking on both obey the same rules (targets only on residues, original id as
    label, untouched positions unchanged) and agree on the replacement pool and, within sampling
    noise, on the selected fraction and the mask / random / keep split."""
    from nanoplm_b200.data.collators import ProtDataCollatorForLM
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    rt, ot = ref.Tokenizer(), ProtTokenizer()
    seqs = _sequences(32, 20, 120, seed=5)
    ex_r = [{"input_ids": torch.tensor(rt.encode(s)), "attention_mask": torch.ones(len(s) + 1, dtype=torch.long)}
            for s in seqs]
    ex_o = [{"input_ids": torch.tensor(ot.encode(s)), "attention_mask": torch.ones(len(s) + 1, dtype=torch.long)}
            for s in seqs]
    rc = ref.collator.ProtDataCollatorForLM(rt, mlm_probability=0.3, mask_token_probability=6,
                                            random_token_probability=3, keep_probability=1)
    oc = ProtDataCollatorForLM(ot, 0.3, mask_token_probability=6, random_token_probability=3, keep_probability=1, seed=4)
    assert abs(rc.p_mask - oc.p_mask) < 1e-12 and abs(rc.p_rand - oc.p_rand) < 1e-12 and abs(rc.p_keep - oc.p_keep) < 1e-12
    assert set(rc.allowed_random_token_ids.tolist()) == set(oc.allowed_random_token_ids.tolist())
    clean = ot.pad(ex_o)["input_ids"]
    special = torch.tensor(sorted(ot.all_special_ids))
    stats = []
    torch.manual_seed(0)
    for coll, ex in ((rc, ex_r), (oc, ex_o)):
        sel = n_mask = n_rand_or_keep = n_changed = n_real = 0
        for _ in range(12):
            out = coll(ex)
            ids, lab, att = out["input_ids"], out["labels"], out["attention_mask"]
            assert ids.dtype == lab.dtype == torch.long and ids.shape == clean.shape
            assert torch.equal(att.long(), (clean != 0).long())
            m = lab != -100
            assert torch.equal(lab[m], clean[m]) and torch.equal(ids[~m], clean[~m])
            assert not torch.isin(clean[m], special).any()
            repl = ids[m]
            assert bool(((repl == 3) | (repl >= 4)).all())
            sel += int(m.sum()); n_real += int((~torch.isin(clean, special)).sum())
            n_mask += int((repl == 3).sum())
            n_changed += int(((repl != 3) & (repl != clean[m])).sum())
        stats.append((sel / n_real, n_mask / sel, n_changed / sel))
    (sr, mr, cr), (so, mo, co) = stats
    assert abs(sr - 0.3) < 0.02 and abs(so - 0.3) < 0.02
    assert abs(mr - 0.6) < 0.03 and abs(mo - 0.6) < 0.03
    # a random draw equals the original id once in 28 times
    assert abs(cr - 0.3 * 27 / 28) < 0.03 and abs(co - 0.3 * 27 / 28) < 0.03
    off_r = ref.collator.ProtDataCollatorForLM(rt, mlm_probability=0.0)(ex_r)
    off_o = ProtDataCollatorForLM(ot, 0.0, seed=0)(ex_o)
    for k in ("input_ids", "attention_mask", "labels"):
        assert torch.equal(off_r[k].long(), off_o[k].long()), k


def test_shard_validation_accepts_and_refuses_the_same_datasets(ref, tmp_path):
    """`validate_pretrain_shards` / `validate_pretrain_dataset` (data/validation.py:182-354): same
    arguments, same shard lists for a good dataset, and a refusal from both for a missing index, an
    index that does not add up to the file size, a wrong shard count and an empty directory."""
    try:
        from nanoplm.data import validation as theirs
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference data modules import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.data import validation as ours
    from nanoplm_b200.data.synthetic import write_synthetic_dataset
    root = write_synthetic_dataset(tmp_path / "ds", 30, 6, 10, 40, samples_per_shard=10)
    a, b = theirs.validate_pretrain_dataset(root), ours.validate_pretrain_dataset(root)
    assert [p.name for p in a["train_shards"]] == [p.name for p in b["train_shards"]] == [
        "shard_0000.bin", "shard_0001.bin", "shard_0002.bin"]
    assert [p.name for p in a["val_shards"]] == [p.name for p in b["val_shards"]]
    assert a["manifest"].train_sequences == b["manifest"].train_sequences == 30
    got = ours.validate_pretrain_shards(root / "train", expected_count=3, check_contents=True)
    assert list(got) == theirs.validate_pretrain_shards(root / "train", expected_count=3, check_contents=True)
    assert len(got) == 3 and got[0].name == "shard_0000.bin" and got["num_sequences"] == 30

    def both_refuse(*args, **kw):
        with pytest.raises(theirs.ValidationError):
            theirs.validate_pretrain_shards(*args, **kw)
        with pytest.raises(ours.ValidationError):
            ours.validate_pretrain_shards(*args, **kw)

    both_refuse(root / "train", expected_count=4)
    both_refuse(root / "nowhere")
    (tmp_path / "empty").mkdir()
    both_refuse(tmp_path / "empty")
    (root / "train" / "shard_0001.idx.npy").rename(root / "train" / "hidden.npy")
    both_refuse(root / "train")
    (root / "train" / "hidden.npy").rename(root / "train" / "shard_0001.idx.npy")
    with open(root / "train" / "shard_0002.bin", "ab") as f:
        f.write(b"\x05\x05")
    both_refuse(root / "train")
    # without the content check only the pairing is looked at, on both sides
    assert len(theirs.validate_pretrain_shards(root / "train", check_contents=False)) == 3
    assert len(ours.validate_pretrain_shards(root / "train", check_contents=False)) == 3


def test_cli_commands_options_and_defaults_cover_the_reference_cli(ref):
    """Every command of the reference's `nanoplm` CLI (cli/__init__.py, cli/data.py, cli/pretrain.py,
    cli/distill.py) exists here, takes every option spelling the reference takes (long and short),
    and has the same defaults, except where listed below with the reason."""
    import click

    from nanoplm_b200.cli import cli as own_cli
    ref_cli, _, _ = _ref_cli_modules()

    def walk(group, prefix=()):
        for name, cmd in group.commands.items():
            if isinstance(cmd, click.Group):
                yield from walk(cmd, prefix + (name,))
            else:
                yield prefix + (name,), cmd

    own = dict(walk(own_cli))
    different_on_purpose = {
        # one pipeline here: the native one is the default, --no-pure-torch selects the HF recipe
        (("pretrain", "run"), "--pure-torch"),
        # the reference declares no usable type / default for it ("auto" is what its config defaults to)
        (("pretrain", "run"), "--num-workers"),
        # parsed as JSON when given; an empty object and "not given" are the same
        (("distill", "run"), "--lr-scheduler-kwargs"),
    }
    seen = 0
    for path, cmd in walk(ref_cli):
        assert path in own, f"command missing: {' '.join(path)}"
        mine = own[path]
        help_names = set(mine.context_settings.get("help_option_names", [])) | set(
            own_cli.context_settings.get("help_option_names", []))
        my_flags, my_by_flag = set(help_names), {}
        for p in mine.params:
            for f in list(p.opts) + list(p.secondary_opts):
                my_flags.add(f)
                my_by_flag[f] = p
        for p in cmd.params:
            if isinstance(p, click.Argument):
                assert any(isinstance(q, click.Argument) and q.name == p.name for q in mine.params), (path, p.name)
                continue
            for f in list(p.opts) + list(p.secondary_opts):
                assert f in my_flags, f"{' '.join(path)}: option {f} missing"
                seen += 1
            flag = p.opts[0]
            if flag in help_names or (path, flag) in different_on_purpose:
                continue
            q = my_by_flag[flag]
            a, b = p.default, q.default
            a = None if a in (0, None) and flag == "--extra-epochs" else a
            b = None if b in (0, None) and flag == "--extra-epochs" else b
            assert a == b or (isinstance(a, float) and abs(a - b) < 1e-12), (path, flag, a, b)
            assert bool(p.required) == bool(q.required), (path, flag)
    assert seen > 150


def test_initialisation_follows_the_reference_distributions(ref):
    """`init_weights` (modeling.py:581-623): N(0, 0.02) embeddings, ones in the norms, U(+-sqrt(3/h))
    for Wqkv / Wi / head.dense, zeros for both output projections and every bias. Different random
    streams, so each tensor is compared by its statistics."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    geom = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2,
                max_position_embeddings=256, mlp_bias=True, attention_bias=True)
    torch.manual_seed(1)
    theirs = ref.Model(ref.Config(**geom)).state_dict()
    torch.manual_seed(2)
    ours = ProtEncoderMLM(ModelConfig(**geom)).state_dict()
    assert set(theirs) == set(ours)
    for k, a in theirs.items():
        a, b = a.float(), ours[k].float()
        assert a.shape == b.shape, k
        if float(a.abs().max()) == 0.0 or float(a.std()) == 0.0:        # zeros / ones: exact
            assert torch.equal(a, b), k
            continue
        assert abs(float(a.std()) - float(b.std())) < 0.08 * float(a.std()) + 1e-4, (k, float(a.std()), float(b.std()))
        assert abs(float(a.mean()) - float(b.mean())) < 0.2 * float(a.std()), k
        if "tok_embeddings" not in k and "decoder" not in k:             # uniform tensors: same support
            assert abs(float(a.abs().max()) - float(b.abs().max())) < 0.02 * float(a.abs().max()), k


def test_training_trajectory_follows_the_reference_recipe(ref):
    """Ten optimizer steps of the reference's recipe, its own pieces on one side (model,
    `_create_optimizer`, `_create_scheduler`, gradient accumulation, clip to 1.0:
    pure_pipeline.py:107-160, 700-790) and this package's on the other (encoder, sharded AdamW engine,
    schedule), from the same weights on the same masked batches: the losses and the gradient norms
    agree step by step and the weights agree at the end."""
    from nanoplm_b200.config.schema import PretrainingConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import schedule
    P = ref.pipeline
    rm, om = _pair(ref)
    rm.train(); om.train()
    cfg = PretrainingConfig(dataset_dir="unused", adam_learning_rate=2e-3, adam_weight_decay=0.05, warmup_ratio=0.2)
    opt = P._create_optimizer(rm, cfg)
    assert [g["weight_decay"] for g in opt.param_groups] == [0.05, 0.0]
    steps, accum = 10, 2
    warm = P._get_warmup_steps(steps, cfg.warmup_ratio)
    sched_r = P._create_scheduler(opt, warm, steps)
    sched_o = schedule.WarmupLinearSchedule(cfg.adam_learning_rate, schedule.get_warmup_steps(steps, cfg.warmup_ratio), steps)
    eng = ShardedEngine(om, AdamWHyper(lr=cfg.adam_learning_rate, beta1=cfg.adam_beta1, beta2=cfg.adam_beta2,
                                       eps=cfg.adam_epsilon, weight_decay=cfg.adam_weight_decay, max_grad_norm=1.0),
                        torch.device("cpu"))
    rt = ref.Tokenizer()
    coll = ref.collator.ProtDataCollatorForLM(rt, mlm_probability=0.3)
    torch.manual_seed(3)
    batches = []
    for i in range(steps * accum):
        seqs = _sequences(6, 10, 70, seed=100 + i)
        batches.append(coll([{"input_ids": torch.tensor(rt.encode(s)),
                              "attention_mask": torch.ones(len(s) + 1, dtype=torch.long)} for s in seqs]))
    for step in range(steps):
        loss_r = loss_o = 0.0
        for k in range(accum):
            b = batches[step * accum + k]
            out = rm(input_ids=b["input_ids"], attention_mask=b["attention_mask"], labels=b["labels"])
            (out["loss"] / accum).backward()
            loss_r += float(out["loss"].detach()) / accum
            out = om(input_ids=b["input_ids"], attention_mask=b["attention_mask"], labels=b["labels"])
            out["loss"].backward()
            loss_o += float(out["loss"].detach()) / accum
        gn_r = float(torch.nn.utils.clip_grad_norm_(rm.parameters(), max_norm=1.0))
        opt.step(); sched_r.step(); opt.zero_grad(set_to_none=True)
        lr = sched_o.get_last_lr()[0]
        gn_o = float(eng.step(lr, grad_accum=accum))
        sched_o.step()
        assert abs(loss_r - loss_o) < 2e-4 * max(1.0, abs(loss_r)), (step, loss_r, loss_o)
        assert abs(gn_r - gn_o) < 1e-3 * gn_r, (step, gn_r, gn_o)
        assert abs(sched_r.get_last_lr()[0] - sched_o.get_last_lr()[0]) < 1e-12
    theirs, ours = rm.state_dict(), om.state_dict()
    worst = max(float((theirs[k].float() - ours[k].float()).abs().max()) for k in theirs)
    assert worst < 5e-4, worst


def test_distillation_trajectory_follows_the_reference_recipe(ref):
    """Eight optimizer steps of the distillation recipe: the reference's student, its trainer's loss
    (distillation/trainer.py:8-40), `AdamW(model.parameters())` (weight decay 0.01 on every tensor,
    distillation/pipeline.py:669), its cosine schedule and the trainer's clipping to 1.0, against this
    package's student, `distillation_loss`, engine and schedule on the same batches."""
    try:
        from nanoplm.distillation.models.student.model import ProtX as RefProtX, ProtXConfig as RefCfg
        from nanoplm.distillation.trainer import DistillationTrainer
        import importlib
        D = importlib.import_module("nanoplm.distillation.pipeline")
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference distillation import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.config.schema import StudentConfig
    from nanoplm_b200.models.student import ProtX
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import schedule
    from nanoplm_b200.runtime.distill import distillation_loss
    torch.manual_seed(0)
    geom = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2)
    rm = RefProtX(RefCfg(**geom)).float()
    with torch.no_grad():
        for p in rm.parameters():
            if p.ndim >= 2:
                p.add_(torch.randn_like(p) * 0.05)
    om = ProtX(StudentConfig(max_position_embeddings=8192, **geom)).float()
    om.load_state_dict(rm.state_dict(), strict=True)
    rm.train(); om.train()
    steps, lr = 8, 2e-3
    opt = torch.optim.AdamW(rm.parameters(), lr=lr)
    sched_r = D._get_scheduler(opt, "cosine", {}, steps)
    sched_o = schedule.make_distill_schedule("cosine", lr, int(steps * 0.05), steps)
    eng = ShardedEngine(om, AdamWHyper(lr=lr, weight_decay=0.01, max_grad_norm=1.0), torch.device("cpu"),
                        compute_dtype=torch.float32, decay_all=True)
    assert all(s.decay for s in eng.slots)
    sd = eng.optimizer_state_dict()
    assert len(sd["param_groups"]) == 1 and len(sd["param_groups"][0]["params"]) == len(list(rm.parameters()))
    assert len(sched_o.state_dict()["base_lrs"]) == len(sched_r.state_dict()["base_lrs"]) == 1
    loss_of = DistillationTrainer._compute_distillation_loss
    tok = rm.tokenizer
    for step in range(steps):
        seqs = _sequences(6, 10, 50, seed=300 + step)
        enc = tok(seqs, padding=True, return_tensors="pt")
        target = torch.randn(enc["input_ids"].shape[0], enc["input_ids"].shape[1], 1024,
                             generator=torch.Generator().manual_seed(step))
        out = rm(enc["input_ids"], enc["attention_mask"], training_mode=True).last_hidden_state
        loss_r = loss_of(None, out, target, enc["attention_mask"])
        loss_r.backward()
        gn_r = float(torch.nn.utils.clip_grad_norm_(rm.parameters(), 1.0))
        opt.step(); sched_r.step(); opt.zero_grad(set_to_none=True)
        batch = {"input_ids": enc["input_ids"], "attention_mask": enc["attention_mask"], "teacher_embeddings": target}
        loss_o = distillation_loss(om, batch)
        loss_o.backward()
        gn_o = float(eng.step(sched_o.get_lr(), grad_accum=1))
        sched_o.step()
        assert abs(float(loss_r.detach()) - float(loss_o.detach())) < 2e-4 * abs(float(loss_r.detach())), step
        assert abs(gn_r - gn_o) < 1e-3 * gn_r, (step, gn_r, gn_o)
        assert abs(sched_r.get_last_lr()[0] - sched_o.get_last_lr()[0]) < 1e-12
    theirs, ours = rm.state_dict(), om.state_dict()
    assert max(float((theirs[k] - ours[k]).abs().max()) for k in theirs) < 5e-4


def test_a_run_moves_between_the_two_pipelines_mid_training(ref, tmp_path, monkeypatch):
    """End to end through both public entry points on one run directory: the reference's
    `run_pure_pretraining` (pure_pipeline.py:334-927) trains 10 steps on a dataset written here and
    saves checkpoints 4 / 8 / 10; this package's `run_pretraining` resumes its checkpoint-4 (same run
    directory, later checkpoints archived, same learning rates, losses that continue the curve) and
    writes 8 / 10; the reference then resumes THAT checkpoint-8 for one more epoch."""
    import json
    import math

    from nanoplm.pretraining.config import PretrainingConfig as RefPre, PureTorchConfig as RefPT, ResumeConfig as RefRes

    from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig, PureTorchConfig, ResumeConfig
    from nanoplm_b200.data.synthetic import write_synthetic_dataset
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.runtime.pretrain import run_pretraining
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    root = write_synthetic_dataset(tmp_path / "ds", 120, 24, 10, 60, samples_per_shard=50)
    geom = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                max_position_embeddings=128)
    common = dict(dataset_dir=str(root), ckp_dir="ckpt", micro_batch_size=8, global_batch_size=8 * 64 * 2,
                  num_epochs=2, logging_steps=1, eval_steps=4, save_steps=4, num_workers=0, bf16=False, tf32=False)

    def ref_model():
        return ref.Model(ref.Config(**geom))

    torch.manual_seed(0)
    ref.pipeline.run_pure_pretraining(ref_model(), RefPre(**common), RefPT(use_compile=False, use_packing=False), None)
    run = next((tmp_path / "ckpt").glob("run-*"))
    files = {"optimizer.pt", "pytorch_model.bin", "rng_state.pth", "scheduler.pt", "training_state.json"}
    assert all({p.name for p in (run / f"checkpoint-{n}").iterdir()} == files for n in (4, 8, 10))
    ref_state = json.loads((run / "checkpoint-4" / "training_state.json").read_text())
    ref_sched = torch.load(run / "checkpoint-8" / "scheduler.pt", weights_only=False)

    res = run_pretraining(ProtEncoderMLM(ModelConfig(**geom), ProtTokenizer()), PretrainingConfig(**common),
                          PureTorchConfig(use_compile=False, use_packing=False),
                          ResumeConfig(True, str(run / "checkpoint-4"), 0))
    assert Path(res["output_dir"]).resolve() == run.resolve() and res["global_step"] == 10
    assert [s for s, _ in res["losses"]] == [5, 6, 7, 8, 9, 10]
    # an untrained model of this size starts at ln(32) = 3.47; the resumed curve starts where the
    # reference's step 4 left it and keeps falling
    assert res["losses"][0][1] < 3.42 and res["losses"][-1][1] < res["losses"][0][1] + 0.02
    archived = [p for p in run.glob("archived_*")]
    assert len(archived) == 1 and sorted(p.name for p in archived[0].iterdir()) == ["checkpoint-10", "checkpoint-8"]
    assert all({p.name for p in (run / f"checkpoint-{n}").iterdir()} >= files for n in (8, 10))
    own_state = json.loads((run / "checkpoint-8" / "training_state.json").read_text())
    assert set(ref_state) <= set(own_state) and own_state["global_step"] == 8
    own_sched = torch.load(run / "checkpoint-8" / "scheduler.pt", weights_only=False)
    assert own_sched["last_epoch"] == ref_sched["last_epoch"] == 8
    assert len(own_sched["base_lrs"]) == len(ref_sched["base_lrs"]) == 2
    assert all(math.isclose(a, b, rel_tol=1e-9) for a, b in zip(own_sched["_last_lr"], ref_sched["_last_lr"]))
    assert (run / ".resume_counter").read_text().strip() == "1"

    # and back: the reference continues from the checkpoint written here, one extra epoch
    ref.pipeline.run_pure_pretraining(ref_model(), RefPre(**common), RefPT(use_compile=False, use_packing=False),
                                      RefRes(True, str(run / "checkpoint-8"), 1))
    assert (run / "checkpoint-15").exists() and (run / ".resume_counter").read_text().strip() == "2"
    final = torch.load(run / "checkpoint-15" / "pytorch_model.bin", weights_only=True)
    mine = torch.load(run / "checkpoint-8" / "pytorch_model.bin", weights_only=True)
    assert set(final) == set(mine)
    moved = max(float((final[k].float() - mine[k].float()).abs().max()) for k in final)
    assert 0 < moved < 0.5


def test_hf_based_reference_model_gives_the_same_logits(ref, tmp_path):
    """The reference's other model class (`ProtModernBertMLM`, models/modern_bert/model.py:43-82: HF's
    `ModernBertForMaskedLM` with the SwiGLU MLP swapped in) has the same state-dict keys as this
    package's encoder, gives the same logits and loss with the same weights, and what its
    `save_pretrained` writes loads here."""
    try:
        from nanoplm.pretraining.models.modern_bert.model import ProtModernBertMLM
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference HF model import failed: {type(exc).__name__}: {exc}")
    from safetensors.torch import load_file

    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    try:
        hf = ProtModernBertMLM(ref.Config(**GEOM)).float().eval()
    except Exception as exc:  # pragma: no cover   (an incompatible transformers version)
        pytest.skip(f"reference HF model does not build here: {type(exc).__name__}: {exc}")
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim >= 2:
                p.add_(torch.randn_like(p) * 0.05)
    om = ProtEncoderMLM(ModelConfig(**GEOM), ProtTokenizer()).float().eval()
    assert set(hf.state_dict()) == set(om.state_dict())
    om.load_state_dict(hf.state_dict(), strict=True)
    tok = ProtTokenizer()
    enc = tok(["MKTAYIAKQRQISFVKSHFSRQ", "ACDEFGHIKLMNPQRSTVWY" * 6, "MK"], padding=True, return_tensors="pt")
    keep = enc["attention_mask"].bool()
    labels = torch.where(keep & (torch.arange(enc["input_ids"].shape[1])[None, :] % 3 == 0), enc["input_ids"],
                         torch.full_like(enc["input_ids"], -100))
    with torch.no_grad():
        theirs = hf(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)
        mine = om(enc["input_ids"], enc["attention_mask"])["logits"]
        mine_loss = om(enc["input_ids"], enc["attention_mask"], labels=labels)["loss"]
    assert (theirs.logits[keep] - mine[keep]).abs().max().item() < 1e-4
    assert abs(float(theirs.loss) - float(mine_loss)) < 1e-4 * max(1.0, float(theirs.loss))
    # save_pretrained stores the tied decoder weight once; the file loads through the tied-key alias
    hf.save_pretrained(tmp_path / "hf")
    sd = load_file(str(tmp_path / "hf" / "model.safetensors"))
    fresh = ProtEncoderMLM(ModelConfig(**GEOM), ProtTokenizer()).float().eval()
    missing = fresh.load_state_dict(sd, strict=False)
    assert not missing.unexpected_keys and set(missing.missing_keys) <= {"decoder.weight", "model.embeddings.tok_embeddings.weight"}
    with torch.no_grad():
        again = fresh(enc["input_ids"], enc["attention_mask"])["logits"]
    assert (again[keep] - mine[keep]).abs().max().item() < 1e-6


def test_download_and_extract_steps_behave_like_the_reference(ref, tmp_path):
    """`Downloader` / `Extractor` (data/downloader.py:16-68, data/extractor.py:14-41): the same bytes
    from the same URL and archive, and an `ExtractionError` from both for a file that is not gzip and
    for an archive cut off in the middle."""
    import gzip

    try:
        from nanoplm.data import downloader as ref_dl
        from nanoplm.data import extractor as ref_ex
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference data modules import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.data import prep
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    fasta = write_synthetic_fasta(tmp_path / "src" / "x.fasta", 300, 20, 200, seed=9)
    raw = Path(fasta).read_bytes()
    gz = tmp_path / "src" / "x.fasta.gz"
    with gzip.open(gz, "wb") as f:
        f.write(raw)
    url = gz.as_uri()
    ref_dl.Downloader(url, tmp_path / "a" / "x.fasta.gz").download()
    prep.Downloader(url, tmp_path / "b" / "x.fasta.gz").download()
    assert (tmp_path / "a" / "x.fasta.gz").read_bytes() == (tmp_path / "b" / "x.fasta.gz").read_bytes() == gz.read_bytes()
    with pytest.raises(Exception):
        ref_dl.Downloader((tmp_path / "nothing.gz").as_uri(), tmp_path / "a" / "n.gz").download()
    with pytest.raises(prep.DownloadError):
        prep.Downloader((tmp_path / "nothing.gz").as_uri(), tmp_path / "b" / "n.gz").download()

    ref_ex.Extractor(tmp_path / "a" / "x.fasta.gz", tmp_path / "a" / "x.fasta").extract()
    prep.Extractor(tmp_path / "b" / "x.fasta.gz", tmp_path / "b" / "x.fasta").extract()
    assert (tmp_path / "a" / "x.fasta").read_bytes() == (tmp_path / "b" / "x.fasta").read_bytes() == raw
    (tmp_path / "plain.gz").write_bytes(raw[:4000])
    (tmp_path / "cut.gz").write_bytes(gz.read_bytes()[: gz.stat().st_size // 2])
    for bad in ("plain.gz", "cut.gz"):
        with pytest.raises(ref_ex.ExtractionError):
            ref_ex.Extractor(tmp_path / bad, tmp_path / "a" / "bad.fasta").extract()
        with pytest.raises(prep.ExtractionError):
            prep.Extractor(tmp_path / bad, tmp_path / "b" / "bad.fasta").extract()


def test_teacher_preprocessing_and_collator_keys_match(ref):
    """`ProtT5.preprocess` (teacher/prott5.py:67-70) against this package's teacher preprocessing on odd
    inputs, and the batch keys of the pre-computed distillation collator (distillation/collator.py:40-60)."""
    try:
        from nanoplm.distillation.collator import DistillDataCollator as RefCollator
        from nanoplm.distillation.models.teacher.prott5 import ProtT5 as RefProtT5
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference distillation import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.data.tokenizer import TeacherTokenizer
    from nanoplm_b200.models.teacher import ProtT5
    from nanoplm_b200.runtime.distill import DistillDataCollator
    theirs, ours = RefProtT5(device="cpu"), ProtT5(device="cpu", random_init=True)
    for s in ("MKTAYIAK", " mkUzob \n", "", "ACDEFGHIKLMNPQRSTVWYX", "a", "BZ*-", None):
        assert theirs.preprocess(s) == ours.preprocess(s) == TeacherTokenizer.preprocess(s or ""), repr(s)
    feats = [{"input_ids": torch.randint(3, 27, (16,), dtype=torch.int8), "attention_mask": torch.ones(16, dtype=torch.int8),
              "teacher_embeddings": torch.randn(16, 1024).half()} for _ in range(3)]
    a = RefCollator(teacher_model=None, on_the_fly=False)(feats)
    b = DistillDataCollator(False, 16)(feats)
    assert set(a) == set(b) == {"input_ids", "attention_mask", "teacher_embeddings"}
    for k in a:
        assert a[k].shape == b[k].shape and torch.equal(a[k].float(), b[k].float()), k


def test_on_the_fly_distillation_targets_match_the_reference_collator(ref):
    """On-the-fly distillation: the reference computes the teacher embeddings inside its collator
    with HF's `T5EncoderModel` (distillation/collator.py:36-96); here the collator only tokenises and
    the native T5 encoder runs inside the step. Same tiny teacher weights, same sequences: the student
    inputs are identical and the targets agree on every real token."""
    try:
        from transformers import T5Config, T5EncoderModel

        from nanoplm.distillation.collator import DistillDataCollator as RefCollator
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference distillation import failed: {type(exc).__name__}: {exc}")
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.data.tokenizer import StudentTokenizer, TeacherTokenizer
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    from nanoplm_b200.runtime.distill import DistillDataCollator
    torch.manual_seed(0)
    hf = T5EncoderModel(T5Config(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4,
                                 relative_attention_num_buckets=32, relative_attention_max_distance=128,
                                 feed_forward_proj="relu", is_encoder_decoder=False, use_cache=False)).float().eval()
    own = T5EncoderTeacher(TeacherConfig(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4),
                           random_init=False).float()
    own.load_state_dict({k: v for k, v in hf.state_dict().items() if k != "encoder.embed_tokens.weight"}, strict=True)
    seqs = _sequences(5, 8, 40, seed=77)
    feats = [{"raw_sequence": s} for s in seqs]
    # the reference's collator calls `batch_encode_plus`, which the installed transformers no longer has on
    # its tokenizers; this package's tokenizers (same ids: test_student_protx_...) still answer to it
    a = RefCollator(teacher_model=hf, teacher_tokenizer=TeacherTokenizer(128), student_tokenizer=StudentTokenizer(),
                    on_the_fly=True, max_seq_len=48)(feats)
    b = DistillDataCollator(True, 48)(feats)
    assert torch.equal(a["input_ids"], b["input_ids"]) and torch.equal(a["attention_mask"], b["attention_mask"])
    with torch.no_grad():
        target = own(b["teacher_input_ids"], b["teacher_attention_mask"], lengths=b["teacher_lengths"])
    keep = b["teacher_attention_mask"].bool()
    assert a["teacher_embeddings"].shape == target.shape
    assert (a["teacher_embeddings"][keep] - target[keep]).abs().max().item() < 2e-4


def test_compat_table_names_exist_in_the_reference_with_compatible_signatures(ref):
    """Every `nanoplm.*` name that `nanoplm_b200.compat` serves exists in the reference under that
    module path (except the few listed, which the reference dropped or never had), and what it resolves
    to here accepts every parameter of the reference's callable, by keyword and, for the required
    ones, in the same position."""
    import importlib
    import inspect

    from nanoplm_b200 import compat
    extras = {("nanoplm", "__version__"), ("nanoplm.cli", "main"), ("nanoplm.pretraining.dataset", "LazyFastaDataset"),
              ("nanoplm.config.datasets", "get_supported_datasets")}

    def params(obj):
        f = obj.__init__ if inspect.isclass(obj) else obj
        try:
            sig = inspect.signature(f)
        except (TypeError, ValueError):
            return None, False
        ps = [p for p in sig.parameters.values() if p.name != "self"]
        return ([p for p in ps if p.kind not in (p.VAR_KEYWORD, p.VAR_POSITIONAL)],
                any(p.kind == p.VAR_KEYWORD for p in ps))

    checked = 0
    for mod_name, table in compat.MODULES.items():
        try:
            theirs_mod = importlib.import_module(mod_name)
        except Exception as exc:                                   # an optional dependency of the reference
            if table:
                pytest.fail(f"reference module {mod_name} does not import: {exc}")
            continue
        for name, target in table.items():
            if (mod_name, name) in extras:
                continue
            assert hasattr(theirs_mod, name), f"{mod_name}.{name} is not a name of the reference"
            theirs = getattr(theirs_mod, name)
            where, _, what = target.partition(":")
            ours = getattr(importlib.import_module(where), what or name)
            if not callable(theirs) or mod_name.endswith(".modeling") or name in ("cli", "logger"):
                continue
            pr, _ = params(theirs)
            po, ours_kwargs = params(ours)
            if pr is None or po is None:
                continue
            own_names = [p.name for p in po]
            for i, p in enumerate(pr):
                assert p.name in own_names or ours_kwargs, f"{mod_name}.{name}: parameter {p.name!r} not accepted here"
                if p.default is inspect.Parameter.empty and p.name in own_names:
                    assert own_names.index(p.name) == i, f"{mod_name}.{name}: {p.name!r} is at another position"
            checked += 1
    assert checked > 45


def test_one_script_runs_on_the_reference_and_on_this_package(ref, tmp_path):
    """A training script written against the reference's Python API (`nanoplm.pretraining.*` imports,
    `run_pure_pretraining(model, PretrainingConfig, PureTorchConfig, ResumeConfig)`) runs unchanged in
    two child processes: with the reference package on the path, and with only
    `nanoplm_b200.compat.install()` in front of it. Both train, save the same checkpoint files and resume."""
    import subprocess
    script = tmp_path / "train.py"
    script.write_text('''
import os, sys, types
os.environ["WANDB_MODE"] = "disabled"
if os.environ.get("USE_COMPAT") == "1":
    import nanoplm_b200.compat
    nanoplm_b200.compat.install()
else:   # optional third-party modules the reference imports without using them here
    for name, attrs in (("IPython", {"get_ipython": lambda: None}), ("h5py", {"File": object}), ("Bio", {}), ("Bio.SeqIO", {})):
        try:
            __import__(name)
        except Exception:
            m = types.ModuleType(name)
            for k, v in attrs.items():
                setattr(m, k, v)
            sys.modules[name] = m
    sys.modules["Bio"].SeqIO = sys.modules["Bio.SeqIO"]
import torch
from pathlib import Path
from nanoplm.pretraining.pure_pipeline import run_pure_pretraining
from nanoplm.pretraining.config import PretrainingConfig, PureTorchConfig, ResumeConfig
from nanoplm.pretraining.models.modern_bert.model import ProtModernBertMLMConfig
from nanoplm.pretraining.models.modern_bert.pure_model import PureProtModernBertMLM
from nanoplm.data.validation import validate_pretrain_dataset
from nanoplm.pretraining.dataset import ShardedDataset

out = sys.argv[1]
info = validate_pretrain_dataset("ds")
assert len(ShardedDataset(data_dir="ds/train")) == info["manifest"].train_sequences == 96
def model():
    torch.manual_seed(0)
    return PureProtModernBertMLM(ProtModernBertMLMConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                                         num_attention_heads=2, max_position_embeddings=64))
cfg = PretrainingConfig(dataset_dir="ds", ckp_dir=out, micro_batch_size=8, global_batch_size=8 * 64 * 2, num_epochs=1,
                        logging_steps=1, eval_steps=2, save_steps=2, num_workers=0, bf16=False, tf32=False)
run_pure_pretraining(model(), cfg, PureTorchConfig(use_compile=False, use_packing=False), None)
run = next(Path(out).glob("run-*"))
cfg.num_epochs = 1
run_pure_pretraining(model(), cfg, PureTorchConfig(use_compile=False, use_packing=False),
                     ResumeConfig(is_resume=True, checkpoint_dir=str(run / "checkpoint-2"), extra_epochs=1))
print("RESULT", sorted(p.name for p in run.iterdir() if p.name.startswith("checkpoint-")),
      sorted(p.name for p in (run / "checkpoint-2").iterdir()))
''')
    from nanoplm_b200.data.synthetic import write_synthetic_dataset
    write_synthetic_dataset(tmp_path / "ds", 96, 16, 10, 60, samples_per_shard=48)
    results = {}
    for arm, path, flag in (("reference", os.pathsep.join([str(REF), str(ROOT)]), "0"), ("compat", str(ROOT), "1")):
        env = dict(os.environ, PYTHONPATH=path, USE_COMPAT=flag, CUDA_VISIBLE_DEVICES="")
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        out = subprocess.run([sys.executable, str(script), f"ckpt_{arm}"], cwd=tmp_path, env=env, capture_output=True,
                             text=True, timeout=900)
        assert out.returncode == 0, f"{arm}: " + (out.stdout + out.stderr)[-3000:]
        results[arm] = [l for l in out.stdout.splitlines() if l.startswith("RESULT")][-1]
    assert results["reference"] == results["compat"], results
    assert "checkpoint-6" in results["compat"] and "optimizer.pt" in results["compat"]


def test_internal_config_knobs_match_the_reference_model(ref):
    """The knobs of the reference's internal `ModernBertConfig` that no YAML exposes
    (modeling.py:39-96): with `norm_bias`, `classifier_bias`, `mlp_bias`, `attention_bias`, the GLU
    MLP variant, a ReLU classifier, another global-attention period and window switched on, the
    reference's `ModernBertForMaskedLM` and this package's encoder have the same keys and, with the same
    weights, the same logits and loss."""
    from nanoplm.pretraining.models.modern_bert import modeling as M

    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    knobs = dict(hidden_size=64, intermediate_size=96, num_hidden_layers=5, num_attention_heads=4, vocab_size=32,
                 max_position_embeddings=256, mlp_activation="glu", hidden_activation="gelu", mlp_bias=True,
                 attention_bias=True, norm_bias=True, classifier_bias=True, classifier_activation="relu",
                 global_attn_every_n_layers=2, local_attention=32, norm_eps=1e-6, decoder_bias=True,
                 global_rope_theta=50000.0, local_rope_theta=5000.0)
    torch.manual_seed(0)
    rm = M.ModernBertForMaskedLM(M.ModernBertConfig(pad_token_id=0, eos_token_id=1, bos_token_id=None, unk_token_id=2,
                                                    mask_token_id=3, **knobs)).float().eval()
    with torch.no_grad():
        for p in rm.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    om = ProtEncoderMLM(ModelConfig(**knobs), ProtTokenizer()).float().eval()
    assert set(om.state_dict()) == set(rm.state_dict())
    assert om.config.layer_types == rm.config.layer_types and om.config.sliding_window == rm.config.sliding_window
    om.load_state_dict(rm.state_dict(), strict=True)
    tok = ProtTokenizer()
    enc = tok(_sequences(4, 30, 120, seed=8), padding=True, return_tensors="pt")
    keep = enc["attention_mask"].bool()
    labels = torch.where(keep & (torch.arange(enc["input_ids"].shape[1])[None, :] % 4 == 1), enc["input_ids"],
                         torch.full_like(enc["input_ids"], -100))
    with torch.no_grad():
        a = rm(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)
        b_logits = om(enc["input_ids"], enc["attention_mask"])["logits"]
        b_loss = om(enc["input_ids"], enc["attention_mask"], labels=labels)["loss"]
    assert (a["logits"][keep] - b_logits[keep]).abs().max().item() < 2e-4 * max(1.0, a["logits"][keep].abs().max().item())
    assert abs(float(a["loss"]) - float(b_loss)) < 2e-4 * max(1.0, float(a["loss"]))
    # logits next to the loss: every position without `sparse_prediction`, the labelled rows only with it
    with torch.no_grad():
        both = om(enc["input_ids"], enc["attention_mask"], labels=labels, return_logits=True)
        assert both["logits"].shape == a["logits"].shape
        assert (a["logits"][keep] - both["logits"][keep]).abs().max().item() < 2e-4 * max(1.0, a["logits"][keep].abs().max().item())
        rs = M.ModernBertForMaskedLM(M.ModernBertConfig(sparse_prediction=True, **knobs)).float().eval()
        rs.load_state_dict(rm.state_dict())
        os_ = ProtEncoderMLM(ModelConfig(sparse_prediction=True, **knobs), ProtTokenizer()).float().eval()
        os_.load_state_dict(rm.state_dict())
        sa = rs(input_ids=enc["input_ids"], attention_mask=enc["attention_mask"], labels=labels)
        sb = os_(enc["input_ids"], enc["attention_mask"], labels=labels, return_logits=True)
    assert sa["logits"].shape == sb["logits"].shape == (int((labels != -100).sum()), 32)
    assert (sa["logits"] - sb["logits"]).abs().max().item() < 2e-4 * max(1.0, sa["logits"].abs().max().item())
    assert abs(float(sa["loss"]) - float(sb["loss"])) < 2e-4 * max(1.0, float(sa["loss"]))
    # every bias starts at zero on both sides
    fresh_r = M.ModernBertForMaskedLM(M.ModernBertConfig(**knobs)).state_dict()
    fresh_o = ProtEncoderMLM(ModelConfig(**knobs), ProtTokenizer()).state_dict()
    for k in fresh_r:
        if k.endswith(".bias"):
            assert float(fresh_r[k].abs().max()) == 0.0 and float(fresh_o[k].abs().max()) == 0.0, k


def test_tokenizer_api_surface_matches(ref, tmp_path):
    """The tokenizer methods user code calls besides encoding (tokenizer.py:8-72, student/tokenizer.py:4-107):
    vocabulary look-ups in both directions, special-token masks, length, BOS mode, `save_vocabulary`."""
    import json

    from nanoplm.distillation.models.student.tokenizer import ProtXTokenizer

    from nanoplm_b200.data.tokenizer import ProtTokenizer, StudentTokenizer
    for theirs, ours in ((ref.Tokenizer(), ProtTokenizer()), (ref.Tokenizer(use_bos_token=True), ProtTokenizer(use_bos_token=True)),
                         (ProtXTokenizer(), StudentTokenizer())):
        assert theirs.get_vocab() == ours.get_vocab() and len(theirs) == len(ours) == ours.vocab_size
        toks = ["A", "L", "X", "<pad>", "</s>", "<unk>", "Q", "not-a-token"]
        assert theirs.convert_tokens_to_ids(toks) == ours.convert_tokens_to_ids(toks)
        assert theirs.convert_tokens_to_ids("W") == ours.convert_tokens_to_ids("W")
        ids = list(range(ours.vocab_size))
        assert theirs.convert_ids_to_tokens(ids) == ours.convert_ids_to_tokens(ids)
        assert theirs.convert_ids_to_tokens(5) == ours.convert_ids_to_tokens(5)
        for name in ("pad_token_id", "eos_token_id", "unk_token_id", "pad_token", "eos_token", "unk_token"):
            assert getattr(theirs, name) == getattr(ours, name), name
        enc = theirs("MKTAYIAKQR")["input_ids"]
        assert enc == ours("MKTAYIAKQR")["input_ids"] == ours.encode("MKTAYIAKQR")
        assert theirs.get_special_tokens_mask(enc, already_has_special_tokens=True) == \
            ours.get_special_tokens_mask(enc, already_has_special_tokens=True)
        assert sorted(theirs.all_special_ids) == sorted(ours.all_special_ids)
        assert theirs.decode(enc, skip_special_tokens=True).replace(" ", "") == ours.decode(enc, skip_special_tokens=True)
    assert ref.Tokenizer(use_bos_token=True)("MK")["input_ids"][0] == ProtTokenizer(use_bos_token=True)("MK")["input_ids"][0] == 29
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    a = ProtXTokenizer().save_vocabulary(str(tmp_path / "a"))
    b = StudentTokenizer().save_vocabulary(str(tmp_path / "b"))
    assert json.loads(Path(a[0]).read_text()) == json.loads(Path(b[0]).read_text()) and Path(a[0]).name == Path(b[0]).name
    ProtTokenizer().save_pretrained(tmp_path / "c")
    assert json.loads((tmp_path / "c" / "vocab.json").read_text()) == ProtTokenizer().get_vocab()
    assert json.loads((tmp_path / "c" / "tokenizer_config.json").read_text())["mask_token"] == "<mask>"
