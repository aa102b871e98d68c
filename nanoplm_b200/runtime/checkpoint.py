"""Checkpoints in the reference's layout (src/nanoplm/pretraining/pure_pipeline.py:235-331):

    <run>/checkpoint-<step>/{pytorch_model.bin, optimizer.pt, scheduler.pt, rng_state.pth,
                             training_state.json}

`pytorch_model.bin` holds the full fp32 state dict under the reference's parameter names (tied
decoder.weight included); `optimizer.pt` is a torch.optim.AdamW state dict with full tensors in the
reference's parameter order. Loading accepts `_orig_mod.`-prefixed keys. Differences: the directory
is written under a temporary name and renamed, so a crash never leaves a half-written checkpoint;
optionally every rank also writes its own optimizer slice (`shard-<rank>.pt` + `index.json`) for a
resume that needs no gather/scatter.

`load_checkpoint` also accepts the layout the reference's HF-Trainer pipeline writes
(src/nanoplm/pretraining/pipeline.py:293-295: `checkpoint-N/{model.safetensors, optimizer.pt,
scheduler.pt, trainer_state.json}`), so a run started there can continue here: the parameter names
are the same (the reference maps them one to one, modeling.py:758-764), the Trainer's AdamW groups
are [decay | no-decay] in `named_parameters` order like this engine's, and the step comes from
`trainer_state.json`. With `hf_files=True` (`pretraining.hf_checkpoint_files`) `save_checkpoint` writes
those two files next to its own, so that the reference's HF-Trainer pipeline (or any safetensors
reader) can pick the run up: `model.safetensors` holds every tensor once (the tied decoder weight is
left to the embedding, as `save_pretrained` does).
"""
from __future__ import annotations

import json
import os
import random
import shutil
from pathlib import Path
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from nanoplm_b200.utils.logging import logger

MODEL_FILE = "pytorch_model.bin"
OPT_FILE = "optimizer.pt"
SCHED_FILE = "scheduler.pt"
RNG_FILE = "rng_state.pth"
STATE_FILE = "training_state.json"


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def save_checkpoint(engine, scheduler, global_step: int, epoch: int, output_dir: str,
                    logging_steps: int, eval_steps: int, save_steps: int, is_main: bool = True,
                    sharded: bool = False, extra_state: Optional[dict] = None, hf_files: bool = False,
                    tied_keys: tuple = ("decoder.weight",)) -> Path:
    final = Path(output_dir) / f"checkpoint-{global_step}"
    tmp = Path(output_dir) / f".tmp-checkpoint-{global_step}"
    model_sd = engine.full_state_dict_model()       # collective
    opt_sd = engine.optimizer_state_dict()          # collective
    if is_main:
        if tmp.exists():
            shutil.rmtree(tmp)
        tmp.mkdir(parents=True, exist_ok=True)
    _barrier()
    if sharded:
        torch.save(engine.shard_state(), tmp / f"shard-{engine.rank}.pt")
    if is_main:
        torch.save(model_sd, tmp / MODEL_FILE)
        torch.save(opt_sd, tmp / OPT_FILE)
        torch.save(scheduler.state_dict(), tmp / SCHED_FILE)
        torch.save({
            "torch_rng": torch.random.get_rng_state(),
            "cuda_rng": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else [],
            "numpy_rng": np.random.get_state(),
            "python_rng": random.getstate(),
        }, tmp / RNG_FILE)
        state = {"global_step": global_step, "epoch": epoch, "logging_steps": logging_steps,
                 "eval_steps": eval_steps, "save_steps": save_steps}
        if extra_state:
            state.update(extra_state)
        (tmp / STATE_FILE).write_text(json.dumps(state, indent=2), encoding="utf-8")
        if hf_files:
            _write_hf_files(tmp, model_sd, global_step, epoch, logging_steps, eval_steps, save_steps, tied_keys)
            _write_hf_config(tmp, getattr(engine.model, "config", None))
        if sharded:
            (tmp / "index.json").write_text(json.dumps(
                {"world_size": engine.world, "total": engine.total, "shard": engine.shard,
                 "files": [f"shard-{r}.pt" for r in range(engine.world)]}, indent=2), encoding="utf-8")
    _barrier()
    if is_main:
        if final.exists():
            shutil.rmtree(final)
        os.replace(tmp, final)
        logger.info(f"Checkpoint saved -> {final}")
    _barrier()
    return final


def _write_hf_files(ckp: Path, model_sd: dict, global_step: int, epoch: int, logging_steps: int,
                    eval_steps: int, save_steps: int, tied_keys: tuple) -> None:
    """`model.safetensors` + `trainer_state.json` as the HF Trainer leaves them (pipeline.py:293-295)."""
    from safetensors.torch import save_file
    tensors = {k: v.detach().to("cpu").contiguous().clone() for k, v in model_sd.items()
               if k not in tied_keys and isinstance(v, torch.Tensor)}
    save_file(tensors, str(ckp / "model.safetensors"), metadata={"format": "pt"})
    trainer_state = {"global_step": int(global_step), "epoch": float(epoch), "max_steps": None,
                     "logging_steps": int(logging_steps), "eval_steps": int(eval_steps),
                     "save_steps": int(save_steps), "log_history": [], "best_metric": None,
                     "best_model_checkpoint": None, "is_world_process_zero": True, "is_local_process_zero": True}
    (ckp / "trainer_state.json").write_text(json.dumps(trainer_state, indent=2), encoding="utf-8")


def _write_hf_config(ckp: Path, cfg) -> None:
    """`config.json` with the field names of HF's `ModernBertConfig`, filled the way the reference's
    HF-based model fills them (models/modern_bert/model.py:52-70), so the directory reads like one
    left by `save_pretrained`. Written as plain JSON: both the per-layer-type fields of recent
    transformers releases (`layer_types`, `rope_parameters`) and the older scalar ones are present."""
    if cfg is None or not hasattr(cfg, "global_attn_every_n_layers"):
        return
    data = {
        "architectures": ["ModernBertForMaskedLM"], "model_type": "modernbert",
        "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
        "num_hidden_layers": cfg.num_hidden_layers, "num_attention_heads": cfg.num_attention_heads,
        "max_position_embeddings": cfg.max_position_embeddings, "hidden_activation": cfg.hidden_activation,
        "initializer_range": cfg.initializer_range, "norm_eps": cfg.norm_eps, "norm_bias": cfg.norm_bias,
        "mlp_bias": cfg.mlp_bias, "mlp_dropout": cfg.mlp_dropout, "attention_bias": cfg.attention_bias,
        "attention_dropout": cfg.attention_dropout, "embedding_dropout": cfg.embedding_dropout,
        "classifier_activation": cfg.classifier_activation, "classifier_bias": cfg.classifier_bias,
        "classifier_pooling": "cls", "decoder_bias": cfg.decoder_bias, "sparse_prediction": cfg.sparse_prediction,
        "sparse_pred_ignore_index": cfg.sparse_pred_ignore_index, "tie_word_embeddings": cfg.tie_word_embeddings,
        "pad_token_id": cfg.pad_token_id, "eos_token_id": cfg.eos_token_id, "bos_token_id": None,
        "unk_token_id": cfg.unk_token_id, "mask_token_id": cfg.mask_token_id, "loss_type": "ForMaskedLM",
        "local_attention": cfg.local_attention, "layer_types": cfg.layer_types,
        "rope_parameters": {"full_attention": {"rope_type": "default", "rope_theta": cfg.global_rope_theta},
                            "sliding_attention": {"rope_type": "default", "rope_theta": cfg.local_rope_theta}},
        "global_attn_every_n_layers": cfg.global_attn_every_n_layers, "global_rope_theta": cfg.global_rope_theta,
        "local_rope_theta": cfg.local_rope_theta, "torch_dtype": "float32",
        # what HF's config has no field for (the MLP variant matters to a loader)
        "nanoplm": {"mlp_activation": cfg.mlp_activation, "norm_type": cfg.norm_type},
    }
    (ckp / "config.json").write_text(json.dumps(data, indent=2), encoding="utf-8")


def load_checkpoint(engine, scheduler, checkpoint_dir: str, restore_rng: bool = True) -> tuple[int, int]:
    ckp = Path(checkpoint_dir)
    if not ckp.exists():
        raise FileNotFoundError(f"Checkpoint directory does not exist: {ckp}")
    index = ckp / "index.json"
    used_shards = False
    if index.exists():
        meta = json.loads(index.read_text())
        mine = ckp / f"shard-{engine.rank}.pt"
        if meta.get("world_size") == engine.world and meta.get("total") == engine.total and mine.exists():
            engine.load_shard_state(torch.load(mine, map_location="cpu", weights_only=True))
            used_shards = True
    if not used_shards:
        model_path = ckp / MODEL_FILE
        hf_path = ckp / "model.safetensors"
        if model_path.exists():
            engine.load_model_state_dict(torch.load(model_path, map_location="cpu", weights_only=True))
        elif hf_path.exists():      # HF-Trainer layout; tied tensors are stored once there
            from safetensors.torch import load_file
            sd = {k: v for k, v in load_file(str(hf_path)).items() if not k.startswith("_")}
            engine.load_model_state_dict(sd)
        else:
            raise FileNotFoundError(f"neither {MODEL_FILE} nor model.safetensors found in {ckp}")
        opt_path = ckp / OPT_FILE
        if opt_path.exists():
            try:
                engine.load_optimizer_state_dict(torch.load(opt_path, map_location="cpu", weights_only=True))
            except Exception as exc:  # truncated / foreign optimizer file: keep the weights, restart moments
                logger.warning(f"Could not load optimizer state ({exc}); optimizer moments start from zero.")
    sched_path = ckp / SCHED_FILE
    if sched_path.exists():
        try:
            scheduler.load_state_dict(torch.load(sched_path, map_location="cpu", weights_only=False))
        except Exception as exc:  # a scheduler pickled by another framework version
            logger.warning(f"Could not load scheduler state ({exc}); the schedule restarts from the loaded step.")
    rng_path = ckp / RNG_FILE
    if restore_rng and rng_path.exists():
        rng = torch.load(rng_path, map_location="cpu", weights_only=False)
        torch.random.set_rng_state(rng["torch_rng"])
        if torch.cuda.is_available() and rng.get("cuda_rng"):
            try:
                torch.cuda.set_rng_state_all(rng["cuda_rng"])
            except Exception:
                pass
        np.random.set_state(rng["numpy_rng"])
        random.setstate(rng["python_rng"])
    state_path = ckp / STATE_FILE
    if state_path.exists():
        st = json.loads(state_path.read_text(encoding="utf-8"))
        return int(st.get("global_step", 0)), int(st.get("epoch", 0))
    hf_state = ckp / "trainer_state.json"
    if hf_state.exists():           # HF Trainer: {"global_step": N, "epoch": fractional epochs done, ...}
        st = json.loads(hf_state.read_text(encoding="utf-8"))
        return int(st.get("global_step", 0)), int(float(st.get("epoch", 0) or 0))
    return 0, 0


def latest_checkpoint(run_dir: str | Path) -> Optional[Path]:
    best, best_step = None, -1
    for d in Path(run_dir).glob("checkpoint-*"):
        try:
            s = int(d.name.split("-")[1])
        except (IndexError, ValueError):
            continue
        # complete = its state file is there (the pretraining pipeline's, or the HF-style one the
        # distillation pipeline writes); checkpoints are renamed into place after their last file
        if s > best_step and ((d / STATE_FILE).exists() or (d / "trainer_state.json").exists()):
            best, best_step = d, s
    return best
