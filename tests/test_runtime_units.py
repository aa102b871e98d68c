"""Schedules, batch arithmetic, run-directory bookkeeping, heartbeat watchdog, sampler fast-forward."""
import math
import os
import time
from pathlib import Path

import pytest
import torch

from nanoplm_b200.runtime.pretrain import ResumableDistributedSampler
from nanoplm_b200.runtime.run_dirs import (archive_future_checkpoints, compute_batch_setup, get_num_workers,
                                           prepare_run_and_steps)
from nanoplm_b200.runtime.schedule import (WarmupLinearSchedule, get_warmup_steps, make_distill_schedule,
                                           num_update_steps_per_epoch)
from nanoplm_b200.runtime.watchdog import Heartbeat, RankFailure, Watchdog, check_or_raise, find_stalled


def test_warmup_linear_schedule_matches_torch_lambda_lr():
    import torch.optim as optim
    from torch.optim.lr_scheduler import LambdaLR
    warm, total = 5, 40
    p = torch.nn.Parameter(torch.zeros(1))
    opt = optim.SGD([p], lr=1e-3)

    def lam(step):
        if step < warm:
            return step / max(1, warm)
        return max(0.0, (total - step) / max(1, total - warm))
    ref = LambdaLR(opt, lam)
    mine = WarmupLinearSchedule(1e-3, warm, total)
    for _ in range(45):
        assert abs(mine.get_lr() - ref.get_last_lr()[0]) < 1e-12
        opt.step()
        ref.step()
        mine.step()
    sd = mine.state_dict()
    other = WarmupLinearSchedule(1e-3, warm, total)
    other.load_state_dict(sd)
    assert other.last_epoch == 45 and other.get_lr() == mine.get_lr()
    other.load_state_dict(ref.state_dict())          # a torch LambdaLR state dict loads as well
    assert other.last_epoch == 45
    assert get_warmup_steps(100, 0.05) == 5 and get_warmup_steps(100, 7) == 7 and get_warmup_steps(101, 0.05) == 6
    assert num_update_steps_per_epoch(10, 4) == 3 and num_update_steps_per_epoch(0, 4) == 1


def test_distillation_schedules():
    for name in ("cosine", "linear", "polynomial", "constant"):
        s = make_distill_schedule(name, 1e-3, 10, 100)
        lrs = []
        for _ in range(100):
            lrs.append(s.get_lr())
            s.step()
        assert lrs[0] == 0 and abs(lrs[10] - 1e-3) < 1e-12 and all(a <= b + 1e-15 for a, b in zip(lrs[:10], lrs[1:11]))
        if name != "constant":
            assert lrs[-1] < 0.1e-3
        else:
            assert lrs[-1] == 1e-3
    with pytest.raises(ValueError):
        make_distill_schedule("bogus", 1e-3, 1, 10)


def test_batch_setup_and_workers():
    b = compute_batch_setup(2 ** 20, 32, 512, 1)
    assert b.grad_accum_steps == 64 and b.global_batch_size_samples == 2048 and b.achieved_global_batch_tokens == 2 ** 20
    assert compute_batch_setup(2 ** 20, 32, 512, 8).grad_accum_steps == 8
    assert compute_batch_setup(1000, 32, 512, 8).grad_accum_steps == 1
    with pytest.raises(ValueError):
        compute_batch_setup(0, 32, 512, 1)
    assert get_num_workers(3, 1) == 3 and get_num_workers("2", 1) == 2 and get_num_workers("auto", 2) >= 1
    with pytest.raises(ValueError):
        get_num_workers(-1, 1)
    with pytest.raises(ValueError):
        get_num_workers("many", 1)


def test_run_naming_resume_counter_and_archive(tmp_path):
    plan = prepare_run_and_steps(str(tmp_path), 3, 10, 50, 100, False, "", None, 1000, 100)
    assert plan.run_name.startswith("run-") and Path(plan.output_dir, "run_name.txt").read_text() == plan.run_name
    assert (plan.logging_steps, plan.eval_steps, plan.save_steps) == (10, 30, 30)      # clamped to total steps
    plan2 = prepare_run_and_steps(str(tmp_path), 3, 10, 50, 100, False, "", None, 1000, 100)
    assert plan2.run_name == plan.run_name + "-2"
    run = Path(plan.output_dir)
    for s in (10, 20, 30):
        (run / f"checkpoint-{s}").mkdir()
    r = prepare_run_and_steps(str(tmp_path), 3, 10, 50, 100, True, str(run / "checkpoint-10"), 2, 1000, 100)
    assert r.run_name == plan.run_name and r.wandb_run_name == plan.run_name + "-re1" and r.num_epochs == 5
    assert r.resume_step == 10 and (run / ".resume_counter").read_text() == "1"
    arch = list(run.glob("archived_*"))
    assert len(arch) == 1 and sorted(p.name for p in arch[0].iterdir()) == ["checkpoint-20", "checkpoint-30"]
    r2 = prepare_run_and_steps(str(tmp_path), 3, 10, 50, 100, True, str(run / "checkpoint-10"), None, 1000, 100)
    assert r2.wandb_run_name.endswith("-re2")
    assert archive_future_checkpoints(run, 10) is None


def test_sampler_partition_and_fast_forward():
    n, world = 103, 4
    seen = []
    for r in range(world):
        s = ResumableDistributedSampler(n, world, r, shuffle=True, seed=5)
        s.set_epoch(2)
        idx = list(s)
        assert len(idx) == math.ceil(n / world)
        seen += idx
    assert set(seen) == set(range(n))
    s = ResumableDistributedSampler(n, world, 1, True, 5)
    s.set_epoch(2)
    full = list(s)
    s.fast_forward(10)
    assert len(s) == len(full) - 10 and list(s) == full[10:]
    assert list(s) == full                                     # the offset applies to one epoch only


def test_heartbeat_and_watchdog(tmp_path):
    hb0 = Heartbeat(tmp_path, 0, interval=0.05).start()
    hb1 = Heartbeat(tmp_path, 1, interval=0.05).start()
    time.sleep(0.15)
    assert find_stalled(tmp_path, 2, max_age=1.0) == []
    assert find_stalled(tmp_path, 3, max_age=1.0) == [2]       # a rank that never joined
    hb1.stop()                                                  # rank 1 "dies" on the host side
    time.sleep(0.4)
    assert find_stalled(tmp_path, 2, max_age=0.3) == [1]
    with pytest.raises(RankFailure) as e:
        check_or_raise(tmp_path, 2, 0.3)
    assert e.value.ranks == [1]
    hb0.stop()


def test_watchdog_sees_a_rank_that_beats_but_makes_no_progress(tmp_path):
    """A rank stuck in a collective keeps its beat thread alive; only its step counter stops."""
    hb0 = Heartbeat(tmp_path, 0, interval=0.05).start()
    hb1 = Heartbeat(tmp_path, 1, interval=0.05).start()
    fired = []
    wd = Watchdog(tmp_path, 2, max_age=5.0, max_step_age=0.4, interval=0.05, on_stall=fired.append).start()
    for step in range(1, 10):          # rank 0 advances, rank 1 stays at step 0 (but keeps beating)
        hb0.step = step
        time.sleep(0.08)
    wd.stop()
    assert fired == [[1]] and wd.fired == [1]
    assert find_stalled(tmp_path, 2, max_age=5.0) == []          # by file age alone nobody is stalled
    hb0.stop()
    hb1.stop()


def test_padding_tail_trim_is_exact_on_cpu():
    """forward(num_real_tokens=...) cuts the padding tail of a static flat batch; loss and gradients of
    the fp32 CPU model must not change."""
    import torch
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    tok = ProtTokenizer()
    model = ProtEncoderMLM(ModelConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                       num_attention_heads=2, max_position_embeddings=128), tok)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            layer.mlp.Wo.weight.normal_(0, 0.05)
    seqs = synthetic_token_sequences(6, 10, 60, seed=3)
    coll = PackingCollator(tok, 64, 0.3, target_rows=10, batch_size=6, seed=3)     # 640 slots, ~200 real
    b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
    n_real = int(b["num_real_tokens"])
    assert n_real + 128 < b["input_ids"].numel()
    keys = ("input_ids", "cu_seqlens", "position_ids", "masked_idx", "masked_labels", "max_seqlen")
    inputs = {k: b[k] for k in keys}
    results = []
    for trim in (None, n_real):
        model.zero_grad()
        out = model(**inputs, num_real_tokens=trim)
        out["loss"].backward()
        results.append((out["loss"].item(), [p.grad.clone() for p in model.parameters() if p.grad is not None]))
    assert abs(results[0][0] - results[1][0]) < 1e-6
    for g0, g1 in zip(results[0][1], results[1][1]):
        assert torch.allclose(g0, g1, atol=1e-6)


def test_checkpoint_with_hf_files_loads_through_the_hf_layout_alone(tmp_path):
    """`hf_files=True` adds model.safetensors + trainer_state.json; with the native files removed the
    directory is exactly what the HF-Trainer pipeline leaves, and it still resumes (weights, step)."""
    import torch
    from safetensors.torch import load_file
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                      max_position_embeddings=64)
    torch.manual_seed(0)
    eng = ShardedEngine(ProtEncoderMLM(cfg, ProtTokenizer()), AdamWHyper(), torch.device("cpu"))
    eng.main_grad.normal_()
    eng.step(1e-3, 1)
    path = ckpt.save_checkpoint(eng, WarmupLinearSchedule(1e-3, 1, 10), 7, 2, str(tmp_path), 1, 5, 5, hf_files=True)
    st = load_file(str(path / "model.safetensors"))
    full = eng.full_state_dict_model()
    assert "decoder.weight" in full and "decoder.weight" not in st          # tied weight stored once
    assert set(st) == set(full) - {"decoder.weight"}
    import json
    assert json.loads((path / "trainer_state.json").read_text())["global_step"] == 7
    # config.json with the field names of HF's ModernBertConfig
    hf_cfg = json.loads((path / "config.json").read_text())
    assert hf_cfg["model_type"] == "modernbert" and hf_cfg["architectures"] == ["ModernBertForMaskedLM"]
    assert (hf_cfg["hidden_size"], hf_cfg["num_hidden_layers"], hf_cfg["vocab_size"], hf_cfg["pad_token_id"]) == (32, 1, 32, 0)
    assert hf_cfg["layer_types"] == ["full_attention"] and hf_cfg["local_attention"] == 128
    assert hf_cfg["nanoplm"]["mlp_activation"] == "swiglu" and hf_cfg["global_rope_theta"] == 160000.0
    assert hf_cfg["rope_parameters"]["sliding_attention"]["rope_theta"] == 10000.0
    for name in ("pytorch_model.bin", "training_state.json", "rng_state.pth"):
        (path / name).unlink()
    torch.manual_seed(1)
    eng2 = ShardedEngine(ProtEncoderMLM(cfg, ProtTokenizer()), AdamWHyper(), torch.device("cpu"))
    step, epoch = ckpt.load_checkpoint(eng2, WarmupLinearSchedule(1e-3, 1, 10), str(path))
    assert (step, epoch) == (7, 2)
    other = eng2.full_state_dict_model()
    for k, v in full.items():
        assert torch.equal(v, other[k]), k


def test_checkpoint_written_from_a_compiled_module_loads(tmp_path):
    """The reference saves the compiled wrapper's state dict when `use_compile` is on, so every key
    carries an `_orig_mod.` prefix (pure_pipeline.py:56-58, 257); such a file resumes here, and so does
    one that stores only one of the two tied embedding / decoder entries."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                      max_position_embeddings=64)
    torch.manual_seed(0)
    src = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for p in src.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    eng = ShardedEngine(src, AdamWHyper(), torch.device("cpu"))
    eng.main_grad.normal_()
    eng.step(1e-3, 1)
    path = ckpt.save_checkpoint(eng, WarmupLinearSchedule(1e-3, 1, 10), 1, 0, str(tmp_path), 1, 5, 5)
    plain = torch.load(path / "pytorch_model.bin", weights_only=True)
    for variant, sd in (("prefixed", {"_orig_mod." + k: v for k, v in plain.items()}),
                        ("decoder only", {k: v for k, v in plain.items() if k != "model.embeddings.tok_embeddings.weight"}),
                        ("embedding only", {k: v for k, v in plain.items() if k != "decoder.weight"})):
        torch.save(sd, path / "pytorch_model.bin")
        torch.manual_seed(1)
        dst = ProtEncoderMLM(cfg, ProtTokenizer())
        eng2 = ShardedEngine(dst, AdamWHyper(), torch.device("cpu"))
        step, _ = ckpt.load_checkpoint(eng2, WarmupLinearSchedule(1e-3, 1, 10), str(path))
        a, b = eng.full_state_dict_model(), eng2.full_state_dict_model()
        assert step == 1 and set(a) == set(b), variant
        assert all(torch.equal(a[k], b[k]) for k in a), variant
        assert dst.decoder.weight.data_ptr() == dst.model.embeddings.tok_embeddings.weight.data_ptr(), variant


def test_measured_peaks_and_mfu(tmp_path, monkeypatch):
    """MFU against the H100 figure the reference hard-codes (pure_pipeline.py:79-82, 803-806) and against
    the bf16 throughput measured on this pool (the fallback figures when the file is absent or unreadable)."""
    from nanoplm_b200.runtime.metrics import H100_PEAK_TFLOPS, MetricsSink
    from nanoplm_b200.utils import peaks
    p = peaks.measured_peaks()
    assert p["source"] in ("measured", "fallback") and p["hbm_gbs"] > 1000 and p["bf16_tflops"] > 100
    monkeypatch.setattr(peaks, "__file__", str(tmp_path / "a" / "b" / "peaks.py"))
    assert peaks.measured_peaks() == peaks.FALLBACK
    (tmp_path / "MEASURED_PEAKS.json").write_text("{not json")
    assert peaks.measured_peaks()["source"] == "fallback"
    (tmp_path / "MEASURED_PEAKS.json").write_text('{"hbm_gbs": 7000.0, "bf16_tflops": 1600.0}')
    assert peaks.measured_peaks() == {"hbm_gbs": 7000.0, "bf16_tflops": 1600.0, "source": "measured"}
    assert H100_PEAK_TFLOPS == 989.4
    monkeypatch.setenv("WANDB_MODE", "disabled")
    sink = MetricsSink(str(tmp_path), "proj", "run", {}, True)
    h100, b200 = sink.mfu(raw_tokens_per_sec=1.0e6, flops_per_token=10 ** 9, world=2)
    assert abs(h100 - 0.5e15 / 989.4e12) < 1e-12 and 0 < b200 < h100     # the B200 denominator is the larger one
    sink.finish(str(tmp_path))


def test_metrics_sink_with_a_stand_in_for_wandb(tmp_path, monkeypatch):
    """The W&B side of the metrics sink against a recording stand-in module: project / run name / config
    at init, `train/global_step` as the x axis (reference: pure_pipeline.py:607-623), every payload
    forwarded, the run id written at the end, and a failing backend that never stops training
    (pure_pipeline.py:828-833)."""
    import json
    import sys
    import types

    from nanoplm_b200.runtime.metrics import MetricsSink
    calls = []
    fake = types.ModuleType("wandb")
    fake.run = None

    def init(**kw):
        calls.append(("init", kw))
        fake.run = types.SimpleNamespace(id="abc123")
    fake.init = init
    fake.define_metric = lambda *a, **kw: calls.append(("define_metric", a, kw))
    fake.log = lambda payload: calls.append(("log", dict(payload)))
    fake.finish = lambda: calls.append(("finish",))
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.setenv("WANDB_MODE", "online")
    sink = MetricsSink(str(tmp_path), "proj", "run-01010101-re2", {"lr": 1e-3}, is_main=True)
    assert calls[0] == ("init", {"project": "proj", "name": "run-01010101-re2", "config": {"lr": 1e-3}})
    assert ("define_metric", ("train/global_step",), {}) in calls
    assert ("define_metric", ("*",), {"step_metric": "train/global_step", "step_sync": True}) in calls
    sink.log({"train/global_step": 1, "train/loss": 2.5})
    assert calls[-1] == ("log", {"train/global_step": 1, "train/loss": 2.5})
    line = json.loads((tmp_path / "metrics.jsonl").read_text().splitlines()[-1])
    assert line["train/loss"] == 2.5 and "time" in line

    def broken(payload):
        raise RuntimeError("network down")
    fake.log = broken
    sink.log({"train/global_step": 2, "train/loss": 2.4})           # swallowed; the backend is dropped
    assert sink.wandb is None and len((tmp_path / "metrics.jsonl").read_text().splitlines()) == 2
    sink.finish(str(tmp_path))
    assert not (tmp_path / "wandb_run_id.txt").exists()

    healthy = MetricsSink(str(tmp_path), "proj", "run", {}, is_main=True)
    healthy.finish(str(tmp_path))
    assert (tmp_path / "wandb_run_id.txt").read_text() == "abc123" and calls[-1] == ("finish",)
    n = len(calls)
    other_rank = MetricsSink(str(tmp_path), "proj", "run", {}, is_main=False)
    other_rank.log({"train/global_step": 3})
    assert len(calls) == n and other_rank.jsonl_path is None         # only the main rank talks to W&B / the file

    def no_init(**kw):
        raise RuntimeError("no credentials")
    fake.init = no_init
    assert MetricsSink(str(tmp_path), "proj", "run", {}, is_main=True).wandb is None


def test_pipeline_with_muon_optimizers_and_configuration_refusals(tmp_path, monkeypatch):
    """`run_pretraining` in one process on the CPU with `optimizer: muon / normuon` (reference:
    pure_pipeline.py:107-147, optim.py:121-184; logs `train/muon_lr` next to the AdamW rate,
    pure_pipeline.py:766-772, 825-827), and the settings it refuses before training starts."""
    import json
    from pathlib import Path

    from nanoplm_b200.config.schema import ModelConfig, PretrainingConfig, PureTorchConfig
    from nanoplm_b200.data.synthetic import write_synthetic_dataset
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.runtime.pretrain import run_pretraining
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("WANDB_MODE", "disabled")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    root = write_synthetic_dataset(tmp_path / "ds", 64, 16, 10, 60, samples_per_shard=32)
    geom = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, max_position_embeddings=64)

    def cfg(**kw):
        base = dict(dataset_dir=str(root), ckp_dir="ck", micro_batch_size=8, global_batch_size=8 * 64, num_epochs=2,
                    logging_steps=1, eval_steps=100, save_steps=100, num_workers=0, bf16=False)
        base.update(kw)
        return PretrainingConfig(**base)

    def model():
        torch.manual_seed(0)
        return ProtEncoderMLM(ModelConfig(**geom), ProtTokenizer())

    for opt in ("muon", "normuon"):
        res = run_pretraining(model(), cfg(optimizer=opt, ckp_dir=f"ck_{opt}", muon_learning_rate=0.02, adam_learning_rate=1e-3,
                                           muon_use_polar_express=(opt == "normuon")),
                              PureTorchConfig(use_packing=True, target_packed_rows=3))
        losses = [l for _, l in res["losses"]]
        assert len(losses) == 8 and losses[-1] < losses[0]
        lines = [json.loads(l) for l in (Path(res["output_dir"]) / "metrics.jsonl").read_text().splitlines()]
        rates = [(l["train/adamw_lr"], l["train/muon_lr"]) for l in lines if "train/muon_lr" in l]
        assert len(rates) == 8 and all(abs(m - 20 * a) < 1e-12 for a, m in rates)          # one schedule, two base rates
        assert (Path(res["output_dir"]) / "checkpoint-8" / "optimizer.pt").exists()
    with pytest.raises(ValueError, match="Invalid optimizer"):
        run_pretraining(model(), cfg(optimizer="sgd"))
    with pytest.raises(ValueError, match="must divide the number of ranks"):
        run_pretraining(model(), cfg(expert_parallel_size=2))
    with pytest.raises(ValueError, match="fp8_recipe"):
        run_pretraining(model(), cfg(fp8=True, fp8_recipe="per_tensor"))
