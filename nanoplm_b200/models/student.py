"""ProtX distillation student: the encoder without the MLM head, followed by an optional
projection to the teacher width and a T5-style (RMS) norm
(reference: src/nanoplm/distillation/models/student/model.py:50-109). Parameter names follow the
reference / HF ModernBertModel (`embeddings.*`, `layers.N.*`, `final_norm`, `proj`, `proj_norm`)."""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanoplm_b200.config.schema import StudentConfig
from nanoplm_b200.data.tokenizer import StudentTokenizer
from nanoplm_b200.models.encoder import (BatchContext, EncoderModel, Linear, Norm,
                                         position_ids_from_cu_seqlens)


class ProtX(EncoderModel):
    def __init__(self, cfg: StudentConfig, tokenizer: Optional[StudentTokenizer] = None):
        self.tokenizer = tokenizer or StudentTokenizer()
        self.student_config = cfg
        mc = cfg.to_model_config(self.tokenizer.vocab_size)
        super().__init__(mc)
        self.proj = self.proj_norm = None
        if cfg.projection_layer:
            self.proj = Linear(cfg.hidden_size, cfg.teacher_dim, False)
            self.proj_norm = Norm(cfg.teacher_dim, 1e-6, rms=True)
        self.init_weights()

    @torch.no_grad()
    def init_weights(self) -> None:
        import math
        cfg = self.config
        bound = math.sqrt(3.0 / cfg.hidden_size)
        nn.init.normal_(self.embeddings.tok_embeddings.weight, 0.0, 0.02)
        for layer in self.layers:
            nn.init.uniform_(layer.attn.Wqkv.weight, -bound, bound)
            nn.init.uniform_(layer.attn.Wo.weight, -bound / 4, bound / 4)
            nn.init.uniform_(layer.mlp.Wi.weight, -bound, bound)
            nn.init.uniform_(layer.mlp.Wo.weight, -bound / 4, bound / 4)
        if self.proj is not None:
            nn.init.uniform_(self.proj.weight, -bound, bound)

    def forward(self, input_ids, attention_mask=None, training_mode: bool = False, cu_seqlens=None,
                position_ids=None):
        """Padded (B, S) or flat ids. Returns {"last_hidden_state"} in the input's layout; with
        training_mode the projected + normed states (teacher width)."""
        pad_info = None
        if input_ids.dim() == 2:
            B, S = input_ids.shape
            if attention_mask is None:
                attention_mask = torch.ones_like(input_ids)
            keep = attention_mask.reshape(-1).bool()
            indices = torch.nonzero(keep, as_tuple=False).flatten()
            ids = input_ids.reshape(-1)[indices]
            lens = attention_mask.sum(dim=-1, dtype=torch.int32)
            cu_seqlens = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
            pad_info = (indices, B, S)
        else:
            ids = input_ids
        T = ids.shape[0]
        if position_ids is None:
            position_ids = position_ids_from_cu_seqlens(cu_seqlens, T, ids.device)
        ctx = BatchContext(cu_seqlens.to(ids.device), position_ids.to(ids.device), T)
        x, _ = EncoderModel.forward(self, ids, ctx)
        if training_mode and self.proj is not None:
            x = self.proj_norm(self.proj(x))
        if pad_info is not None:
            indices, B, S = pad_info
            full = torch.zeros((B * S, x.shape[-1]), dtype=x.dtype, device=x.device)
            full = full.index_copy(0, indices, x)
            x = full.view(B, S, -1)
        return {"last_hidden_state": x}

    # ---- utilities of the reference student (model.py:111-497) ---------------------------------
    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def parameter_breakdown(self) -> dict:
        groups = {"embeddings": 0, "attention": 0, "mlp": 0, "norms": 0, "projection": 0, "other": 0}
        for name, p in self.named_parameters():
            if name.startswith("embeddings.tok"):
                groups["embeddings"] += p.numel()
            elif ".attn." in name:
                groups["attention"] += p.numel()
            elif ".mlp." in name:
                groups["mlp"] += p.numel()
            elif "norm" in name:
                groups["norms"] += p.numel()
            elif name.startswith("proj"):
                groups["projection"] += p.numel()
            else:
                groups["other"] += p.numel()
        groups["total"] = sum(groups.values())
        return groups

    @torch.no_grad()
    def embed_sequences(self, sequences: list[str], batch_size: int = 16, per_token: bool = False,
                        device: Optional[torch.device] = None) -> list[torch.Tensor]:
        """Mean-pooled (EOS excluded) or per-token embeddings for raw sequences."""
        device = device or next(self.parameters()).device
        was_training = self.training
        self.eval()
        out = []
        for i in range(0, len(sequences), batch_size):
            enc = self.tokenizer(sequences[i:i + batch_size], padding=True, return_tensors="pt")
            ids, mask = enc["input_ids"].to(device), enc["attention_mask"].to(device)
            h = self(ids, mask)["last_hidden_state"].float()
            for b in range(ids.shape[0]):
                n = int(mask[b].sum()) - 1          # drop the trailing </s>
                out.append(h[b, :n].cpu() if per_token else h[b, :n].mean(0).cpu())
        self.train(was_training)
        return out


def inspect_checkpoint_architecture(path: str | Path) -> dict:
    """Infers the student architecture from a saved state dict (safetensors or torch)."""
    p = Path(path)
    if p.suffix == ".safetensors":
        from safetensors.torch import load_file
        sd = load_file(str(p))
    else:
        sd = torch.load(p, map_location="cpu", weights_only=True)
    layers = sorted({int(k.split(".")[1]) for k in sd if k.startswith("layers.")})
    hidden = sd["embeddings.tok_embeddings.weight"].shape[1]
    info = {"hidden_size": hidden, "vocab_size": sd["embeddings.tok_embeddings.weight"].shape[0],
            "num_hidden_layers": len(layers), "projection_layer": "proj.weight" in sd,
            "num_parameters": sum(v.numel() for v in sd.values())}
    if layers:
        info["intermediate_size"] = sd[f"layers.{layers[0]}.mlp.Wo.weight"].shape[1]
    return info


def calculate_model_parameters(model: torch.nn.Module) -> dict:
    """Total and trainable parameter counts (reference: student/model.py, parameter utilities)."""
    total = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    return {"total": total, "trainable": trainable, "frozen": total - trainable}


def print_parameter_breakdown(model: "ProtX") -> dict:
    """Logs the per-group parameter counts of a student and returns them."""
    from nanoplm_b200.utils.logging import logger
    groups = model.parameter_breakdown()
    total = max(1, groups["total"])
    for name, n in groups.items():
        if name != "total":
            logger.info(f"{name:>12s}: {n:>12,d}  ({100.0 * n / total:5.1f} %)")
    logger.info(f"{'total':>12s}: {groups['total']:>12,d}")
    return groups


def load_and_generate_embeddings(checkpoint: str | Path, sequences: list[str], cfg: Optional[StudentConfig] = None,
                                 batch_size: int = 16, per_token: bool = False,
                                 device: Optional[torch.device] = None) -> list[torch.Tensor]:
    """Loads a saved student (safetensors or torch state dict) and embeds raw sequences: mean-pooled
    over the residues (the trailing </s> excluded) or one vector per residue
    (reference: student/model.py:111-248). Without `cfg` the architecture is inferred from the file;
    the head count defaults to hidden_size / 64."""
    p = Path(checkpoint)
    if p.is_dir():
        p = p / ("model.safetensors" if (p / "model.safetensors").exists() else "pytorch_model.bin")
    if p.suffix == ".safetensors":
        from safetensors.torch import load_file
        sd = load_file(str(p))
    else:
        sd = torch.load(p, map_location="cpu", weights_only=True)
    if cfg is None:
        info = inspect_checkpoint_architecture(p)
        cfg = StudentConfig(hidden_size=info["hidden_size"], intermediate_size=info.get("intermediate_size", 2 * info["hidden_size"]),
                            num_hidden_layers=info["num_hidden_layers"],
                            num_attention_heads=max(1, info["hidden_size"] // 64),
                            projection_layer=info["projection_layer"])
    model = ProtX(cfg)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if unexpected:
        raise KeyError(f"unexpected keys in student checkpoint: {sorted(unexpected)[:5]}")
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = model.to(device)
    if device.type == "cuda":
        model = model.to(torch.bfloat16)
    return model.embed_sequences(sequences, batch_size=batch_size, per_token=per_token, device=device)
