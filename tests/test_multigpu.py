"""Multi-GPU paths: NCCL optimizer step and the P2P-fused optimizer step against a single-GPU run,
and the bounded wait of the peer barrier (a flag nobody sets -> CommTimeout, context still usable)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model():
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256)
    return ProtEncoderMLM(cfg, ProtTokenizer())


def _batches(n):
    from nanoplm_b200.data.collators import PackingCollator
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    tok = ProtTokenizer()
    out = []
    for i in range(n):
        seqs = synthetic_token_sequences(16, 20, 200, seed=50 + i)
        coll = PackingCollator(tok, 256, 0.3, target_rows=10, batch_size=16, seed=i)
        b = coll([{"input_ids": torch.from_numpy(s)} for s in seqs])
        b.pop("num_real_tokens")
        out.append(b)
    return out


def _worker(rank, world, port, fused, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    model = _model()
    if fused == "muon":
        from nanoplm_b200.config.schema import PretrainingConfig
        from nanoplm_b200.parallel.muon import MuonEngine
        eng = MuonEngine(model, AdamWHyper(lr=2e-3, weight_decay=0.01),
                         PretrainingConfig(dataset_dir="x", optimizer="normuon", muon_learning_rate=5e-3), dev)
        assert eng._kernels
        if world > 1:       # even stacks (all-gather) and an uneven one (3 matrices of 256 x 256: all-reduce)
            assert {st.even for st in eng.stacks} == {True, False}
    elif fused == "param_sharded":
        from nanoplm_b200.parallel.param_sharded import ParamShardedEngine
        eng = ParamShardedEngine(model, AdamWHyper(lr=2e-3, weight_decay=0.01), dev, fused_comm=True)
        assert type(eng.fused).__name__ == "ParamShardedStep" and len(eng.gather_states) == 2 * 4 + 1
    else:
        eng = ShardedEngine(model, AdamWHyper(lr=2e-3, weight_decay=0.01), dev, fused_comm=fused)
    if fused is True and world > 1:
        assert eng.fused is not None, "symmetric memory path was expected on this machine"
    model.train()
    st = TrainStep(model, eng, WarmupLinearSchedule(2e-3, 2, 100), dev)
    batches = _batches(12)
    losses = []
    for step in range(6):
        losses.append(st.step_from_host(batches[2 * step:2 * step + 2][rank::world]))
    torch.cuda.synchronize()
    _lib.check_status()
    if fused == "param_sharded":
        # after a step every gathered matrix waits for its next forward GEMM; one forward pass clears them
        assert all(st_.stale for st_ in eng.gather_states)
        with torch.no_grad():
            from nanoplm_b200.runtime.pretrain import model_inputs, move_batch
            model(**model_inputs(move_batch(batches[0], dev)))
        assert not any(st_.stale for st_ in eng.gather_states)
        torch.cuda.synchronize()
        _lib.check_status()
    t = torch.tensor(losses, device=dev)
    if world > 1:
        dist.all_reduce(t)
        t /= world
    sd = eng.full_state_dict_model()
    if rank == 0:
        torch.save({"losses": t.cpu(), "sd": sd, "fused": getattr(eng, "fused", None) is not None}, out_path)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _run(world, fused, out_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fused, out_path)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    return torch.load(out_path)


@pytest.mark.multigpu
def test_two_gpu_steps_match_single_gpu(tmp_path):
    one = _run(1, False, str(tmp_path / "one.pt"))
    nccl = _run(2, False, str(tmp_path / "nccl.pt"))
    fused = _run(2, True, str(tmp_path / "fused.pt"))
    assert fused["fused"] and not nccl["fused"]
    for other in (nccl, fused):
        assert torch.allclose(one["losses"], other["losses"], atol=3e-2), (one["losses"], other["losses"])
    # the two 2-GPU paths compute the same update from the same gradients
    worst = 0.0
    for k in nccl["sd"]:
        a, b = nccl["sd"][k].float(), fused["sd"][k].float()
        worst = max(worst, (a - b).abs().max().item())
    assert worst < 5e-3, worst


@pytest.mark.multigpu
def test_two_gpu_parameter_sharded_training_matches_single_gpu(tmp_path):
    """Row-sharded parameters: the weights' all-gather runs inside the first forward GEMMs of a step
    (RoPE, residual, SwiGLU and GELU epilogues), every rank reduces and updates its own row blocks."""
    one = _run(1, False, str(tmp_path / "one.pt"))
    nccl = _run(2, False, str(tmp_path / "nccl.pt"))
    ps = _run(2, "param_sharded", str(tmp_path / "ps.pt"))
    assert torch.allclose(one["losses"], ps["losses"], atol=3e-2), (one["losses"], ps["losses"])
    worst = 0.0
    for k in nccl["sd"]:
        worst = max(worst, (nccl["sd"][k].float() - ps["sd"][k].float()).abs().max().item())
    assert worst < 5e-3, worst


@pytest.mark.multigpu
def test_matrix_parallel_muon_on_two_gpus_matches_single_gpu(tmp_path):
    """NorMuon with every stack of same-shape matrices split over two GPUs (momentum kernel and
    grouped Newton-Schulz on the owner, all-gather of the bf16 orthogonal factors) against the
    same training on one GPU."""
    one = _run(1, "muon", str(tmp_path / "one.pt"))
    two = _run(2, "muon", str(tmp_path / "two.pt"))
    assert one["losses"][-1] < one["losses"][0] - 0.1, one["losses"]
    # the orthogonalised update has unit scale whatever the gradient's size, so run-to-run differences
    # of the gradients (atomic accumulation order) show up at the size of a step in single elements:
    # compare the losses and the mean deviation of the weights, bound single elements loosely
    assert torch.allclose(one["losses"], two["losses"], atol=5e-2), (one["losses"], two["losses"])
    worst, mean = 0.0, 0.0
    for k in one["sd"]:
        d = (one["sd"][k].float() - two["sd"][k].float()).abs()
        worst, mean = max(worst, d.max().item()), max(mean, d.mean().item())
    assert mean < 4e-3 and worst < 8e-2, (mean, worst)


def test_peer_barrier_times_out_without_hanging():
    """Self-loop: 'peer' 1 is this GPU's own flag array and nothing ever sets its slot."""
    import ctypes
    from ctypes import c_double, c_int, c_uint, c_void_p
    from nanoplm_b200.ops import _lib
    handle = _lib.lib("comm")
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    arr = (c_void_p * 2)(c_void_p(flags.data_ptr()), c_void_p(flags.data_ptr() + 32))
    status = _lib.status_word()
    status.zero_()
    rc = handle.nplm_peer_barrier(arr, c_int(0), c_int(2), c_uint(1), c_double(0.2),
                                  c_void_p(status.data_ptr()), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(_lib.CommTimeout):
        _lib.check_status()
    # the context is still usable and the status word was cleared
    x = torch.ones(4, device="cuda") * 2
    assert x.sum().item() == 8
    _lib.check_status()


def _ep_worker(rank, world, port, out_path):
    """Expert parallelism over peer memory: every rank routes its own tokens to experts that are
    split over the ranks; outputs and gradients must match an fp32 run of all experts on all tokens."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.ops import moe as M
    from test_moe_gpu import _moe_oracle
    BF = torch.bfloat16
    T, E, k, C, I = 700 + 37 * rank, 8, 2, 128, 128
    El = E // world
    g = torch.Generator(device="cpu").manual_seed(7)
    Wi_all = (torch.randn(E, 2 * I, C, generator=g) * 0.06).to(BF).to(dev)
    Wo_all = (torch.randn(E, C, I, generator=g) * 0.06).to(BF).to(dev)
    torch.manual_seed(100 + rank)
    x = torch.randn(T, C, device=dev).to(BF).requires_grad_(True)
    logits = (torch.randn(T, E, device=dev) * 1.5).to(BF).requires_grad_(True)
    gy = torch.randn(T, C, device=dev).to(BF)
    Wi = Wi_all[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    Wo = Wo_all[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    comm = M.MoEComm(C, E, k, group=dist.group.WORLD, capacity_factor=float(world))
    worst = {}
    for it in range(2):                       # second pass reuses the symmetric buffers
        for t in (x, logits, Wi, Wo):
            t.grad = None
        y, aux = M.moe_mlp(x, logits, Wi, Wo, k, comm)
        ((y.float() * gy.float()).sum() + 0.5 * aux).backward()
        torch.cuda.synchronize()
        _lib.check_status()
        # oracle: all experts, this rank's tokens (outputs, dx, dlogits)
        x32 = x.detach().float().requires_grad_(True)
        l32 = logits.detach().float().requires_grad_(True)
        Wi32 = Wi_all.float().requires_grad_(True)
        Wo32 = Wo_all.float().requires_grad_(True)
        experts = M.router_topk(logits.detach(), k)[2]
        y_ref, aux_ref = _moe_oracle(x32, l32, Wi32, Wo32, k, experts)
        ((y_ref * gy.float()).sum() + 0.5 * aux_ref).backward()
        # weight gradients are sums over the tokens of every rank
        gWi, gWo = Wi32.grad.clone(), Wo32.grad.clone()
        dist.all_reduce(gWi)
        dist.all_reduce(gWo)

        def rel(a, b):
            return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)

        worst = {"y": rel(y, y_ref), "dx": rel(x.grad, x32.grad), "dlogits": rel(logits.grad, l32.grad),
                 "dWi": rel(Wi.grad, gWi[rank * El:(rank + 1) * El]),
                 "dWo": rel(Wo.grad, gWo[rank * El:(rank + 1) * El])}
        for name, v in worst.items():
            assert v < 0.06, (it, rank, name, v)
    assert comm.dropped_rows() == 0
    # buffers too small for a router that sends everything to rank 0's experts: the rows past the
    # capacity are dropped and counted, nothing aborts, the result stays finite
    tight = M.MoEComm(C, E, k, group=dist.group.WORLD, capacity_factor=0.5)
    skew = logits.detach().clone()
    skew[:, :El] += 8.0
    skew.requires_grad_(True)
    y2, aux2 = M.moe_mlp(x.detach().requires_grad_(True), skew, Wi, Wo, k, tight)
    ((y2.float() * gy.float()).sum() + 0.5 * aux2).backward()
    torch.cuda.synchronize()
    _lib.check_status()
    lost = torch.tensor([tight.dropped_rows()], device=dev)
    dist.all_reduce(lost)
    assert int(lost.item()) > 0 and torch.isfinite(y2.float()).all() and torch.isfinite(skew.grad.float()).all()
    if rank == 0:
        torch.save(worst, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_expert_parallel_peer_memory(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    out = str(tmp_path / "ep.pt")
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert os.path.exists(out)


def _ag_worker(rank, world, port, out_path):
    """All-gather fused into the GEMM: the weight is row-sharded over the ranks in symmetric memory;
    every rank multiplies its own activations by the whole weight."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.comm.fused_optimizer import SymmetricBuffer
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.ops import kernels as K
    BF = torch.bfloat16
    results = {}
    for (M, N, Kd, epi) in [(1000, 512, 256, K.EPI_STORE), (4096, 3072, 1024, K.EPI_STORE),
                            (2048, 1024, 512, K.EPI_ADD)]:
        g = torch.Generator(device="cpu").manual_seed(11)
        W = (torch.randn(N, Kd, generator=g) * 0.05).to(BF).to(dev)
        torch.manual_seed(200 + rank)
        x = torch.randn(M, Kd, device=dev).to(BF)
        res = torch.randn(M, N, device=dev).to(BF) if epi == K.EPI_ADD else None
        sb = SymmetricBuffer(N * Kd, BF, dev, dist.group.WORLD)
        full = sb.tensor.view(N, Kd)
        rows = N // world
        for it in range(2):                      # second pass: buffers already hold the gathered matrix
            full.fill_(float("nan"))
            full[rank * rows:(rank + 1) * rows] = W[rank * rows:(rank + 1) * rows]
            flags = torch.zeros(8, dtype=torch.int32, device=dev)
            torch.cuda.synchronize()
            dist.barrier()                       # every rank's shard is in place
            y = K.gemm_ag(x, full, sb.ptr_array, rank, world, flags, epi=epi, aux=res)
            torch.cuda.synchronize()
            _lib.check_status()
            dist.barrier()                       # peers are done reading before the next fill
            ref = x.float() @ W.float().t()
            if res is not None:
                ref = ref + res.float()
            err = (y.float() - ref).abs().max().item() / ref.abs().max().item()
            assert err < 0.02, (M, N, Kd, it, err)
            assert torch.equal(full, W), "the local buffer must hold the gathered weight"
            results[(M, N, Kd)] = err
    if rank == 0:
        torch.save(results, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_all_gather_gemm(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    out = str(tmp_path / "ag.pt")
    procs = [ctx.Process(target=_ag_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert os.path.exists(out)


def _moe_train_worker(rank, world, port, out_path):
    """MoE encoder trained for a few steps: world 1 = replicated experts on one GPU; world 2 = experts
    split over the GPUs through ExpertParallelEngine and the peer-memory dispatch."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.config.schema import ModelConfig, MoEConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.ops import _lib
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.parallel.expert_engine import ExpertParallelEngine, shard_model_experts
    from nanoplm_b200.runtime.pretrain import TrainStep
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      max_position_embeddings=256,
                      moe=MoEConfig(num_experts=8, top_k=2, expert_intermediate_size=128, every_n_layers=2))
    model = ProtEncoderMLM(cfg, ProtTokenizer())
    with torch.no_grad():
        for layer in model.model.layers:
            layer.attn.Wo.weight.normal_(0, 0.03)
            if hasattr(layer.mlp, "Wo"):
                layer.mlp.Wo.weight.normal_(0, 0.03)
            else:
                layer.mlp.experts_Wo.normal_(0, 0.03)
    hyper = AdamWHyper(lr=2e-3, weight_decay=0.01)
    if world > 1:
        assert shard_model_experts(model, dist.group.WORLD) == 1
        eng = ExpertParallelEngine(model, hyper, dev, fused_comm=True)   # dense part on the peer-memory step
    else:
        eng = ShardedEngine(model, hyper, dev)
    model.train()
    st = TrainStep(model, eng, WarmupLinearSchedule(2e-3, 2, 100), dev)
    batches = _batches(8)
    losses = []
    for step in range(4):
        losses.append(st.step_from_host(batches[2 * step:2 * step + 2][rank::world]))
    torch.cuda.synchronize()
    _lib.check_status()
    t = torch.tensor(losses, device=dev)
    if world > 1:
        dist.all_reduce(t)
        t /= world
    sd = eng.full_state_dict_model()
    if rank == 0:
        torch.save({"losses": t.cpu(), "sd": sd}, out_path)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.multigpu
def test_expert_parallel_training_on_two_gpus(tmp_path):
    ctx = mp.get_context("spawn")
    res = {}
    for world in (1, 2):
        port = _free_port()
        out = str(tmp_path / f"moe{world}.pt")
        procs = [ctx.Process(target=_moe_train_worker, args=(r, world, port, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            assert p.exitcode == 0, f"rank exited with {p.exitcode}"
        res[world] = torch.load(out)
    assert torch.allclose(res[1]["losses"], res[2]["losses"], atol=4e-2), (res[1]["losses"], res[2]["losses"])
    assert res[2]["losses"][-1] < res[2]["losses"][0]
    for k, v in res[1]["sd"].items():
        assert res[2]["sd"][k].shape == v.shape, k


def _ag_fp8_worker(rank, world, port, out_path):
    """fp8 all-gather GEMM: e4m3 weight rows and their block scales are sharded over the ranks."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.comm.fused_optimizer import SymmetricBuffer
    from nanoplm_b200.ops import _lib, fp8
    BF = torch.bfloat16
    for (M, N, Kd) in [(1000, 512, 256), (4096, 3072, 1024)]:
        g = torch.Generator(device="cpu").manual_seed(11)
        W = (torch.randn(N, Kd, generator=g) * 0.05).to(BF).to(dev)
        torch.manual_seed(300 + rank)
        x = torch.randn(M, Kd, device=dev).to(BF)
        qx = fp8.quant_rows(x)
        qw = fp8.quant_tile(W, transpose=False, block=True)       # every rank quantises the same W
        rows, nb = N // world, N // 128 // world
        pay = SymmetricBuffer(N * Kd, torch.uint8, dev, dist.group.WORLD)
        sc = SymmetricBuffer((Kd // 128) * (N // 128), torch.float32, dev, dist.group.WORLD)
        payload, scales = pay.tensor.view(N, Kd), sc.tensor.view(Kd // 128, N // 128)
        payload.fill_(0x7f)                                         # NaN pattern in e4m3
        scales.fill_(float("nan"))
        payload[rank * rows:(rank + 1) * rows] = qw.q[rank * rows:(rank + 1) * rows]
        scales[:, rank * nb:(rank + 1) * nb] = qw.scale[:, rank * nb:(rank + 1) * nb]
        flags = torch.zeros(8, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        y = fp8.gemm_fp8_ag(qx, payload, pay.ptr_array, scales, sc.ptr_array, rank, world, flags)
        torch.cuda.synchronize()
        _lib.check_status()
        dist.barrier()
        ref = fp8.gemm_fp8(qx, qw)
        assert torch.equal(payload, qw.q) and torch.equal(scales, qw.scale)
        assert torch.equal(y, ref), (M, N, Kd, (y.float() - ref.float()).abs().max().item())
    if rank == 0:
        torch.save({"ok": True}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_all_gather_gemm_fp8(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    out = str(tmp_path / "agf8.pt")
    procs = [ctx.Process(target=_ag_fp8_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0, f"rank exited with {p.exitcode}"
    assert os.path.exists(out)


def _stats_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from nanoplm_b200.comm.peer_stats import PeerStats
    ps = PeerStats.try_create(dev)
    assert ps is not None and ps.world == world
    got = []
    for call in range(5):      # alternating tables, a different number of values every call
        vals = [float(rank + 1) * (call + 1), 1000.0 + rank, 0.25 * (rank + 1) + call][: 1 + call % 3]
        got.append(ps.all_reduce(vals, max_mask=0b100))
    if rank == 0:
        torch.save(got, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.multigpu
def test_peer_stats_all_reduce_two_gpus(tmp_path):
    out = str(tmp_path / "stats.pt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_stats_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    got = torch.load(out)
    for call, res in enumerate(got):
        want = [3.0 * (call + 1), 2001.0, 0.5 + call][: 1 + call % 3]      # sum, sum, max over ranks 0 and 1
        assert res == pytest.approx(want), (call, res, want)


def test_peer_stats_single_process():
    """One process: the table lives in ordinary device memory and the kernel talks to itself."""
    from nanoplm_b200.comm.peer_stats import PeerStats
    ps = PeerStats.try_create(torch.device("cuda:0"))
    for call in range(3):
        vals = [1.5 + call, 7.0, -2.0]
        assert ps.all_reduce(vals, max_mask=0b010) == pytest.approx(vals)
    with pytest.raises(ValueError):
        ps.all_reduce([0.0] * 17)
