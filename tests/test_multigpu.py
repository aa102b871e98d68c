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
    eng = ShardedEngine(model, AdamWHyper(lr=2e-3, weight_decay=0.01), dev, fused_comm=fused)
    if fused and world > 1:
        assert eng.fused is not None, "symmetric memory path was expected on this machine"
    model.train()
    st = TrainStep(model, eng, WarmupLinearSchedule(2e-3, 2, 100), dev)
    batches = _batches(12)
    losses = []
    for step in range(6):
        losses.append(st.step_from_host(batches[2 * step:2 * step + 2][rank::world]))
    torch.cuda.synchronize()
    _lib.check_status()
    t = torch.tensor(losses, device=dev)
    if world > 1:
        dist.all_reduce(t)
        t /= world
    sd = eng.full_state_dict_model()
    if rank == 0:
        torch.save({"losses": t.cpu(), "sd": sd, "fused": eng.fused is not None}, out_path)
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
