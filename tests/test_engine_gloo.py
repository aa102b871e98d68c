"""Sharded engine over CPU ranks (gloo): 2-rank training must follow the 1-rank trajectory, and
checkpoints written by a sharded run must load in a single-process run (and vice versa)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make_model():
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                      max_position_embeddings=128)
    m = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for layer in m.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            layer.mlp.Wo.weight.normal_(0, 0.05)
    return m


def _batches(n):
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    tok = ProtTokenizer()
    out = []
    for i in range(n):
        seqs = synthetic_token_sequences(8, 10, 60, seed=100 + i)
        coll = PackingCollator(tok, 64, 0.3, target_rows=8, batch_size=8, seed=i)
        b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
        b.pop("num_real_tokens")
        out.append(b)
    return out


def _train(rank, world, port, tmp, result_q):
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _make_model()
    eng = ShardedEngine(model, AdamWHyper(lr=5e-3, weight_decay=0.01), torch.device("cpu"))
    sch = WarmupLinearSchedule(5e-3, 2, 100)
    st = TrainStep(model, eng, sch, "cpu")
    batches = _batches(8)
    losses = []
    for step in range(4):
        mine = batches[2 * step:2 * step + 2][rank::world]     # each rank takes its share of 2 micro-batches
        losses.append(st.step_from_host(mine))
    if world > 1:
        t = torch.tensor(losses)
        dist.all_reduce(t)
        losses = (t / world).tolist()
    ckpt.save_checkpoint(eng, sch, 4, 0, tmp, 1, 10, 10, is_main=rank == 0, sharded=world > 1)
    sd = eng.full_state_dict_model()
    if rank == 0:
        torch.save((world, losses, {k: v.clone() for k, v in sd.items()}), os.path.join(tmp, "result.pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _run(world, tmp):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_train, args=(r, world, port, tmp, None)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    return torch.load(os.path.join(tmp, "result.pt"))


def test_two_rank_training_matches_single_rank(tmp_path):
    d1, d2 = str(tmp_path / "w1"), str(tmp_path / "w2")
    os.makedirs(d1)
    os.makedirs(d2)
    _, l1, sd1 = _run(1, d1)
    _, l2, sd2 = _run(2, d2)
    for a, b in zip(l1, l2):
        assert abs(a - b) < 1e-4, (l1, l2)
    for k in sd1:
        assert torch.allclose(sd1[k], sd2[k], atol=2e-5), k
    # files of the reference layout exist, plus the per-rank shards of the sharded run
    for name in ("pytorch_model.bin", "optimizer.pt", "scheduler.pt", "rng_state.pth", "training_state.json"):
        assert os.path.exists(os.path.join(d2, "checkpoint-4", name))
    assert os.path.exists(os.path.join(d2, "checkpoint-4", "shard-1.pt"))
    assert os.path.exists(os.path.join(d2, "checkpoint-4", "index.json"))

    # a checkpoint written by 2 ranks resumes in 1 process (full-tensor path) with identical state
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    model = _make_model()
    eng = ShardedEngine(model, AdamWHyper(lr=5e-3, weight_decay=0.01), torch.device("cpu"))
    sch = WarmupLinearSchedule(5e-3, 2, 100)
    step, epoch = ckpt.load_checkpoint(eng, sch, os.path.join(d2, "checkpoint-4"))
    assert (step, epoch) == (4, 0) and eng.step_count == 4 and sch.last_epoch == 4
    sd = eng.full_state_dict_model()
    for k in sd1:
        assert torch.allclose(sd[k], sd2[k], atol=1e-7), k
    opt = torch.load(os.path.join(d2, "checkpoint-4", "optimizer.pt"))
    assert len(opt["param_groups"]) == 2 and opt["param_groups"][1]["weight_decay"] == 0.0
    n_params = sum(len(g["params"]) for g in opt["param_groups"])
    assert n_params == len(eng.slots) and len(opt["state"]) == n_params


def _make_moe_model():
    from nanoplm_b200.config.schema import ModelConfig, MoEConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2,
                      max_position_embeddings=128,
                      moe=MoEConfig(num_experts=4, top_k=2, expert_intermediate_size=32, every_n_layers=2))
    m = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for layer in m.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            if hasattr(layer.mlp, "Wo"):
                layer.mlp.Wo.weight.normal_(0, 0.05)
            else:
                layer.mlp.experts_Wo.normal_(0, 0.05)
    return m


def _train_moe(rank, world, port, tmp, expert_parallel, per_step=2, ep_size=None):
    """world == 1: replicated experts, gradient accumulation over the step's micro-batches.
    world == 2 + expert_parallel: every rank takes one micro-batch and owns half of the experts.
    ep_size < world: world / ep_size expert-parallel groups, every group holds every expert once."""
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.parallel.expert_engine import ExpertParallelEngine, make_expert_groups, shard_model_experts
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _make_moe_model()
    hyper = AdamWHyper(lr=5e-3, weight_decay=0.01, max_grad_norm=0.5)
    if expert_parallel:
        ep_group, edp_group = make_expert_groups(ep_size or world)
        assert shard_model_experts(model, ep_group) == 1
        eng = ExpertParallelEngine(model, hyper, torch.device("cpu"), ep_group=ep_group, edp_group=edp_group)
    else:
        eng = ShardedEngine(model, hyper, torch.device("cpu"))
    st = TrainStep(model, eng, WarmupLinearSchedule(5e-3, 2, 100), "cpu")
    batches = _batches(3 * per_step + 2)
    losses = []
    for step in range(3):
        losses.append(st.step_from_host(batches[per_step * step:per_step * step + per_step][rank::world]))
    if world > 1:
        t = torch.tensor(losses)
        dist.all_reduce(t)
        losses = (t / world).tolist()
    sd = eng.full_state_dict_model()
    opt = eng.optimizer_state_dict()
    if rank == 0:
        torch.save((losses, {k: v.clone() for k, v in sd.items()}, opt.get("expert_parallel")),
                   os.path.join(tmp, "result.pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _run_moe(world, tmp, expert_parallel, per_step=2, ep_size=None):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_train_moe, args=(r, world, port, tmp, expert_parallel, per_step, ep_size))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    return torch.load(os.path.join(tmp, "result.pt"))


def test_expert_parallel_training_matches_replicated_experts(tmp_path):
    """Experts split over 2 ranks (rank-local AdamW, shared clipping norm, rows exchanged between
    ranks) must follow the single-process trajectory with all experts in one place."""
    d1, d2 = str(tmp_path / "one"), str(tmp_path / "ep")
    os.makedirs(d1)
    os.makedirs(d2)
    l1, sd1, _ = _run_moe(1, d1, False)
    l2, sd2, extra = _run_moe(2, d2, True)
    for a, b in zip(l1, l2):
        assert abs(a - b) < 2e-4, (l1, l2)
    assert set(sd1) == set(sd2)
    for k in sd1:
        assert sd1[k].shape == sd2[k].shape, k            # gathered experts have the full first axis
        assert torch.allclose(sd1[k], sd2[k], atol=5e-5), k
    assert extra is not None and all(v.shape[0] == 4 for v in extra["exp_avg"].values())


def test_two_expert_parallel_groups_of_two_ranks_match_replicated_experts(tmp_path):
    """Four ranks as two expert-parallel groups (expert_parallel_size 2): rows travel inside a group, the
    replicas of an expert in the two groups sum their gradients, the clipping norm counts every expert
    once. Same trajectory as one process with all experts and the four micro-batches of a step."""
    d1, d2 = str(tmp_path / "one"), str(tmp_path / "ep")
    os.makedirs(d1)
    os.makedirs(d2)
    l1, sd1, _ = _run_moe(1, d1, False, per_step=4)
    l2, sd2, extra = _run_moe(4, d2, True, per_step=4, ep_size=2)
    for a, b in zip(l1, l2):
        assert abs(a - b) < 2e-4, (l1, l2)
    assert set(sd1) == set(sd2)
    for k in sd1:
        assert sd1[k].shape == sd2[k].shape, k
        assert torch.allclose(sd1[k], sd2[k], atol=5e-5), k
    assert extra is not None and all(v.shape[0] == 4 for v in extra["exp_avg"].values())


def _train_muon(rank, world, port, tmp, optimizer):
    from nanoplm_b200.config.schema import PretrainingConfig
    from nanoplm_b200.parallel.engine import AdamWHyper
    from nanoplm_b200.parallel.muon import MuonEngine
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _make_model()
    cfg = PretrainingConfig(dataset_dir="x", optimizer=optimizer, bf16=False)
    eng = MuonEngine(model, AdamWHyper(lr=1e-3, weight_decay=0.01), cfg, torch.device("cpu"))
    sch = WarmupLinearSchedule(1e-3, 2, 100)
    st = TrainStep(model, eng, sch, "cpu")
    batches = _batches(8)
    for step in range(3):
        st.step_from_host(batches[2 * step:2 * step + 2][rank::world])
    opt_sd = eng.optimizer_state_dict()          # collective: momentum comes from the owning rank
    sd = eng.full_state_dict_model()
    # a 2-layer model has 2 matrices per shape: with 2 ranks every rank owns one of each
    owned = sum(st_.hi - st_.lo for st_ in eng.stacks)
    if rank == 0:
        torch.save((sd, opt_sd, owned, len(eng.muon_slots)), os.path.join(tmp, "muon.pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("optimizer", ["muon", "normuon"])
def test_matrix_parallel_muon_matches_single_rank(tmp_path, optimizer):
    """Two ranks each orthogonalise half of every stack of same-shape matrices and exchange the
    orthogonal factors; parameters, momentum and NorMuon row moments must equal the 1-rank run."""
    out = []
    for world in (1, 2):
        d = str(tmp_path / f"w{world}")
        os.makedirs(d)
        ctx = mp.get_context("spawn")
        port = _free_port()
        procs = [ctx.Process(target=_train_muon, args=(r, world, port, d, optimizer)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        out.append(torch.load(os.path.join(d, "muon.pt")))
    (sd1, opt1, owned1, n1), (sd2, opt2, owned2, n2) = out
    assert owned1 == n1 and owned2 < n2
    for k in sd1:
        assert torch.allclose(sd1[k], sd2[k], atol=3e-5), k
    for i in opt1["state"]:
        assert torch.allclose(opt1["state"][i]["exp_avg"], opt2["state"][i]["exp_avg"], atol=3e-5), i
    if optimizer == "normuon":
        for k, v in opt1["normuon_row_second_moment"].items():
            assert torch.allclose(v, opt2["normuon_row_second_moment"][k], atol=1e-5), k


def _make_wide_model():
    """256-wide: every layer matrix splits into whole 128-row tiles over two ranks."""
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=128)
    m = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for layer in m.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.05)
            layer.mlp.Wo.weight.normal_(0, 0.05)
    return m


def _train_param_sharded(rank, world, port, tmp, sharded):
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.parallel.param_sharded import ParamShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    if world > 1:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    model = _make_wide_model()
    cls = ParamShardedEngine if sharded else ShardedEngine
    eng = cls(model, AdamWHyper(lr=3e-3, weight_decay=0.01), torch.device("cpu"))
    if sharded:
        n_blocks = sum(1 for p in eng.pieces if p.gathered)
        assert n_blocks == 2 * 2 * 4 + 2            # 4 matrices per layer + the head's dense, two row blocks each
        assert all((p.b - p.a) * 2 == p.slot.numel for p in eng.pieces if p.gathered)
        owned = sum(p.b - p.a for p in eng.mine)
        assert owned < 0.6 * eng.total              # about half of the parameters live here
    st = TrainStep(model, eng, WarmupLinearSchedule(3e-3, 2, 100), "cpu")
    batches = _batches(40)
    losses = []
    for step in range(20):
        losses.append(st.step_from_host(batches[2 * step:2 * step + 2][rank::world]))
    if world > 1:
        t = torch.tensor(losses)
        dist.all_reduce(t)
        losses = (t / world).tolist()
    ckpt.save_checkpoint(eng, st.scheduler, 20, 0, tmp, 1, 100, 100, is_main=rank == 0)
    sd = eng.full_state_dict_model()
    opt = eng.optimizer_state_dict()
    if rank == 0:
        torch.save((losses, {k: v.clone() for k, v in sd.items()}, opt), os.path.join(tmp, "result.pt"))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def test_parameter_sharded_engine_follows_the_single_rank_trajectory(tmp_path):
    """Row-block ownership of parameters / optimizer state over two ranks: 20 steps give the losses,
    weights and Adam moments of the single-process run, and its checkpoint loads in a plain engine."""
    out = []
    for world, sharded in ((1, False), (2, True)):
        d = str(tmp_path / f"w{world}")
        os.makedirs(d)
        ctx = mp.get_context("spawn")
        port = _free_port()
        procs = [ctx.Process(target=_train_param_sharded, args=(r, world, port, d, sharded)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
            assert p.exitcode == 0
        out.append(torch.load(os.path.join(d, "result.pt")))
    (l1, sd1, opt1), (l2, sd2, opt2) = out
    assert l1[-1] < l1[0] - 0.05
    for a, b in zip(l1, l2):
        assert abs(a - b) < 2e-4, (l1, l2)
    for k in sd1:
        assert torch.allclose(sd1[k], sd2[k], atol=5e-5), k
    for i in opt1["state"]:
        assert torch.allclose(opt1["state"][i]["exp_avg_sq"], opt2["state"][i]["exp_avg_sq"], atol=1e-6), i
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    eng = ShardedEngine(_make_wide_model(), AdamWHyper(lr=3e-3, weight_decay=0.01), torch.device("cpu"))
    step, _ = ckpt.load_checkpoint(eng, WarmupLinearSchedule(3e-3, 2, 100), str(tmp_path / "w2" / "checkpoint-20"))
    assert step == 20
    back = eng.full_state_dict_model()
    for k in sd2:
        assert torch.allclose(back[k], sd2[k], atol=1e-7), k
