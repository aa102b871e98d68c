"""Failure detection with CPU ranks (gloo): a rank that raises between steps is noticed by the
others through a short process-group timeout instead of an endless wait; a truncated optimizer file
does not block resuming. Nothing here touches a GPU."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                       # step 1: everyone is alive
    assert t[0].item() == world
    if rank == 1:
        # host-side failure between steps: this rank leaves without joining the next collective
        os._exit(17)
    try:
        dist.all_reduce(t)                   # step 2: must fail within the timeout, not hang
        outcome = "completed"
    except Exception as exc:                 # noqa: BLE001
        outcome = f"error:{type(exc).__name__}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)


def test_lost_rank_surfaces_as_an_error_not_a_hang(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 3, port, str(tmp_path))) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode is not None, "a surviving rank hung"
    assert procs[1].exitcode == 17
    for r in (0, 2):
        assert (tmp_path / f"rank{r}.txt").read_text().startswith("error:")


def test_truncated_optimizer_file_does_not_block_resume(tmp_path):
    from nanoplm_b200.config.schema import ModelConfig
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    from nanoplm_b200.models.encoder import ProtEncoderMLM
    from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine
    from nanoplm_b200.runtime import checkpoint as ckpt
    from nanoplm_b200.runtime.schedule import WarmupLinearSchedule
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                      max_position_embeddings=64)
    torch.manual_seed(0)
    m = ProtEncoderMLM(cfg, ProtTokenizer())
    eng = ShardedEngine(m, AdamWHyper(), torch.device("cpu"))
    eng.main_grad.normal_()
    eng.step(1e-3, 1)
    sch = WarmupLinearSchedule(1e-3, 1, 10)
    path = ckpt.save_checkpoint(eng, sch, 1, 0, str(tmp_path), 1, 5, 5)
    assert not list(tmp_path.glob(".tmp-*"))                         # written under a temp name, then renamed
    opt = path / "optimizer.pt"
    opt.write_bytes(opt.read_bytes()[:100])                          # simulate a crash while copying
    m2 = ProtEncoderMLM(cfg, ProtTokenizer())
    eng2 = ShardedEngine(m2, AdamWHyper(), torch.device("cpu"))
    step, _ = ckpt.load_checkpoint(eng2, WarmupLinearSchedule(1e-3, 1, 10), str(path))
    a, b = eng.full_state_dict_model(), eng2.full_state_dict_model()
    assert step == 1 and all(torch.allclose(a[k], b[k]) for k in a) and eng2.exp_avg.abs().sum() == 0
    assert ckpt.latest_checkpoint(tmp_path).name == "checkpoint-1"
    with pytest.raises(FileNotFoundError):
        ckpt.load_checkpoint(eng2, sch, str(tmp_path / "checkpoint-99"))
