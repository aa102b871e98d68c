"""ModernBERT-style bidirectional encoder for protein MLM on packed (T, C) activations.

Behaviour follows the reference model (src/nanoplm/pretraining/models/modern_bert/modeling.py):
embedding -> LayerNorm; pre-norm blocks whose first layer has no attention norm (:408-412); fused
Wqkv, RoPE with theta 160000 on global layers and 10000 on sliding-window layers (:468-491);
global attention on every third layer, +-64 window elsewhere (:93-96); SwiGLU MLP with
[value | gate] = Wi(x) (:300-302); final norm; head = norm(act(dense(x))) (:547-559); decoder tied
to the embedding, with bias (:571-579); zero-initialised output projections (:581-623). Parameter
names equal the reference's, so `pytorch_model.bin` files are interchangeable.

Differences by design: activations are always flat `(T, C)` with `cu_seqlens` (padded input is
unpadded on entry); the MLM head runs only on positions that carry a label, which leaves the loss
unchanged; optional varlen depthwise conv, hyper-connections (mHC) and MoE blocks.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanoplm_b200.config.schema import ModelConfig
from nanoplm_b200.ops import functional as ops


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    def forward(self, x, residual=None, act=None):
        return ops.linear(x, self.weight, self.bias, residual=residual, act=act)


class Norm(nn.Module):
    def __init__(self, dim: int, eps: float, rms: bool = False, bias: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        # the optional bias (`norm_bias`, off in every reference recipe) is a plain add after the kernel
        self.bias = nn.Parameter(torch.zeros(dim)) if bias else None
        self.eps, self.rms = eps, rms

    def forward(self, x):
        y = ops.norm(x, self.weight, self.eps, self.rms)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def with_residual(self, x):
        """(norm(x), x): the second value is the skip connection of a pre-norm block."""
        y, skip = ops.norm_residual(x, self.weight, self.eps, self.rms)
        return (y if self.bias is None else y + self.bias.to(y.dtype)), skip


class Embeddings(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size, padding_idx=cfg.pad_token_id)
        self.norm = Norm(cfg.hidden_size, cfg.norm_eps, cfg.norm_type == "rmsnorm", cfg.norm_bias)
        self.p_drop = float(cfg.embedding_dropout)

    def forward(self, ids):
        x = ops.embed_norm(ids, self.tok_embeddings.weight, self.norm.weight, self.norm.eps, self.norm.rms)
        if self.norm.bias is not None:
            x = x + self.norm.bias.to(x.dtype)
        if self.p_drop > 0.0 and self.training:     # reference: modeling.py:220-223
            x = F.dropout(x, self.p_drop, True)
        return x


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.num_heads, self.head_dim = cfg.num_attention_heads, cfg.head_dim
        self.scale = self.head_dim ** -0.5
        self.Wqkv = Linear(cfg.hidden_size, 3 * cfg.hidden_size, cfg.attention_bias)
        self.Wo = Linear(cfg.hidden_size, cfg.hidden_size, cfg.attention_bias)

    def forward(self, x, ctx: "BatchContext", window: int, rope: tuple, residual=None):
        H, D = self.num_heads, self.head_dim
        fused = (x.is_cuda and x.dtype == torch.bfloat16 and D == 64 and self.Wqkv.bias is None
                 and x.dim() == 2 and self.Wqkv.in_features % 8 == 0 and not ops.fp8_enabled())
        if fused:   # RoPE in the QKV GEMM epilogue, its transpose inside the attention backward
            qkv = ops.linear_rope(x, self.Wqkv.weight, ctx.position_ids, rope[0], rope[1], 2 * H * D)
            if self.Wo.bias is None:
                return ops.attention_out_proj(qkv, self.Wo.weight, residual, ctx.seq_start, ctx.seq_end, H, D,
                                              window, self.scale, rope=(ctx.position_ids, rope[0], rope[1]))
            y = ops.attention_varlen(qkv, ctx.seq_start, ctx.seq_end, H, D, window, self.scale,
                                     rope=(ctx.position_ids, rope[0], rope[1]))
        else:
            qkv = self.Wqkv(x)
            qkv = ops.rope_qkv(qkv, ctx.position_ids, rope[0], rope[1], H, D)
            y = ops.attention_varlen(qkv, ctx.seq_start, ctx.seq_end, H, D, window, self.scale)
        return self.Wo(y, residual=residual)


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, intermediate: Optional[int] = None):
        super().__init__()
        inter = intermediate or cfg.intermediate_size
        self.swiglu = cfg.mlp_activation == "swiglu"
        self.hidden_activation = cfg.hidden_activation
        self.Wi = Linear(cfg.hidden_size, 2 * inter, cfg.mlp_bias)
        self.Wo = Linear(inter, cfg.hidden_size, cfg.mlp_bias)
        self.p_drop = float(cfg.mlp_dropout)

    def forward(self, x, residual=None):
        drop = self.p_drop > 0.0 and self.training
        if self.swiglu and self.Wi.bias is None and self.Wo.bias is None and not drop:
            return ops.mlp_swiglu(x, self.Wi.weight, self.Wo.weight, residual)
        if self.swiglu:
            h = self.Wi(x, act="swiglu")
        else:  # GLU variant: act(value) * gate (reference: modeling.py:281-282)
            v, g = self.Wi(x).chunk(2, dim=-1)
            h = ops.activation(v.contiguous(), self.hidden_activation) * g
        if drop:    # between the activation and the down-projection (reference: modeling.py:277, 298)
            h = F.dropout(h, self.p_drop, True)
        return self.Wo(h, residual=residual)


class BatchContext:
    """Per-batch device metadata shared by all layers."""

    def __init__(self, cu_seqlens: torch.Tensor, position_ids: torch.Tensor, T: int):
        self.cu_seqlens = cu_seqlens
        self.position_ids = position_ids.to(torch.int32)
        self.seq_start, self.seq_end = ops.seq_bounds(cu_seqlens, T)
        self.T = T


class EncoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.attention_type = cfg.layer_types[layer_idx]
        rms = cfg.norm_type == "rmsnorm"
        self.attn_norm = nn.Identity() if layer_idx == 0 else Norm(cfg.hidden_size, cfg.norm_eps, rms, cfg.norm_bias)
        self.attn = Attention(cfg)
        self.mlp_norm = Norm(cfg.hidden_size, cfg.norm_eps, rms, cfg.norm_bias)
        self.is_moe = cfg.is_moe_layer(layer_idx)
        if self.is_moe:
            from .moe import MoEMLP
            self.mlp = MoEMLP(cfg)
        else:
            self.mlp = MLP(cfg)
        self.conv = None
        if cfg.conv_kernel_size > 0:
            from .conv import VarlenDepthwiseConv
            self.conv = VarlenDepthwiseConv(cfg.hidden_size, cfg.conv_kernel_size, cfg.conv_bias)
        self.mhc_attn = self.mhc_mlp = None
        if cfg.mhc_streams > 1:
            from .mhc import HyperConnection
            self.mhc_attn = HyperConnection(cfg.hidden_size, cfg.mhc_streams, cfg.mhc_sinkhorn_iters, cfg.norm_eps)
            self.mhc_mlp = HyperConnection(cfg.hidden_size, cfg.mhc_streams, cfg.mhc_sinkhorn_iters, cfg.norm_eps)

    def _attn_branch(self, h, ctx, window, rope, residual, normed: bool = False):
        if not normed:
            h = self.attn_norm(h)
        if self.conv is not None:
            h = h + self.conv(h, ctx)
        return self.attn(h, ctx, window, rope, residual=residual)

    def forward(self, x, ctx: BatchContext, window: int, rope: tuple):
        aux = None
        if self.mhc_attn is None:
            if isinstance(self.attn_norm, Norm):
                h, skip = self.attn_norm.with_residual(x)
                x = self._attn_branch(h, ctx, window, rope, residual=skip, normed=True)
            else:
                x = self._attn_branch(x, ctx, window, rope, residual=x)
            if self.is_moe:
                y, aux = self.mlp(self.mlp_norm(x))
                x = x + y
            else:
                h, skip = self.mlp_norm.with_residual(x)
                x = self.mlp(h, residual=skip)
            return x, aux
        # hyper-connections: x is (T, n, C)
        h, state = self.mhc_attn.read(x)
        x = self.mhc_attn.write(x, self._attn_branch(h, ctx, window, rope, residual=None), state)
        h, state = self.mhc_mlp.read(x)
        if self.is_moe:
            y, aux = self.mlp(self.mlp_norm(h))
        else:
            y = self.mlp(self.mlp_norm(h))
        x = self.mhc_mlp.write(x, y, state)
        return x, aux


class EncoderModel(nn.Module):
    """Embeddings + layers + final norm; forward takes flat ids and a BatchContext."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.config = cfg
        self.embeddings = Embeddings(cfg)
        self.layers = nn.ModuleList([EncoderLayer(cfg, i) for i in range(cfg.num_hidden_layers)])
        self.final_norm = Norm(cfg.hidden_size, cfg.norm_eps, cfg.norm_type == "rmsnorm", cfg.norm_bias)
        self._rope_cache: dict = {}

    def rope(self, device) -> dict:
        key = str(device)
        if key not in self._rope_cache:
            c = self.config
            self._rope_cache[key] = {
                "full_attention": ops.rope_tables(c.max_position_embeddings, c.head_dim, c.global_rope_theta, device),
                "sliding_attention": ops.rope_tables(c.max_position_embeddings, c.head_dim, c.local_rope_theta, device),
            }
        return self._rope_cache[key]

    def forward_hidden(self, input_ids, ctx: BatchContext):
        """Returns the residual stream after the last layer (before final_norm) and MoE aux loss."""
        cfg = self.config
        x = self.embeddings(input_ids)
        rope = self.rope(x.device)
        n = cfg.mhc_streams
        if n > 1:
            x = x.unsqueeze(1).expand(-1, n, -1).contiguous()
        aux_total = None
        for layer in self.layers:
            lt = layer.attention_type
            window = -1 if lt == "full_attention" else cfg.sliding_window
            x, aux = layer(x, ctx, window, rope[lt])
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        if n > 1:
            x = x.sum(dim=1)
        return x, aux_total

    def forward(self, input_ids, ctx: BatchContext):
        x, aux = self.forward_hidden(input_ids, ctx)
        return self.final_norm(x), aux


class PredictionHead(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.dense = Linear(cfg.hidden_size, cfg.hidden_size, cfg.classifier_bias)
        self.norm = Norm(cfg.hidden_size, cfg.norm_eps, cfg.norm_type == "rmsnorm", cfg.norm_bias)
        self.act = cfg.classifier_activation

    def forward(self, x):
        if self.act == "gelu":
            return self.norm(self.dense(x, act="gelu"))
        return self.norm(ops.activation(self.dense(x), self.act))


def position_ids_from_cu_seqlens(cu_seqlens: torch.Tensor, total: int, device=None) -> torch.Tensor:
    """[0,3,5,9] -> [0,1,2, 0,1, 0,1,2,3] (positions restart at every sequence)."""
    device = device or cu_seqlens.device
    cu = cu_seqlens.to(device=device, dtype=torch.int64)
    lens = cu[1:] - cu[:-1]
    starts = torch.repeat_interleave(cu[:-1], lens, output_size=total)
    return (torch.arange(total, device=device) - starts).to(torch.int32)


class ProtEncoderMLM(nn.Module):
    """Masked-LM model. `forward` accepts the reference's three input conventions
    (modeling.py:631-752): flat packed ids + cu_seqlens + position_ids; padded (B, S) ids with an
    attention mask (optionally with collator-provided cu_seqlens); returns {"loss", "logits"}."""

    _tied_weights_keys = {"decoder.weight": "model.embeddings.tok_embeddings.weight"}

    def __init__(self, cfg: ModelConfig, tokenizer=None):
        super().__init__()
        self.config = cfg
        self.tokenizer = tokenizer
        self.model = EncoderModel(cfg)
        self.head = PredictionHead(cfg)
        self.decoder = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=cfg.decoder_bias)
        self.init_weights()
        if cfg.tie_word_embeddings:
            self.decoder.weight = self.model.embeddings.tok_embeddings.weight

    @torch.no_grad()
    def init_weights(self) -> None:
        cfg = self.config
        bound = math.sqrt(3.0 / cfg.hidden_size)
        emb_std = float(cfg.initializer_range) if cfg.tie_word_embeddings else 1.0
        nn.init.normal_(self.model.embeddings.tok_embeddings.weight, 0.0, emb_std)
        for m in self.modules():
            if isinstance(m, Norm):
                nn.init.ones_(m.weight)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
        for layer in self.model.layers:
            nn.init.uniform_(layer.attn.Wqkv.weight, -bound, bound)
            nn.init.zeros_(layer.attn.Wo.weight)
            lins = [layer.attn.Wqkv, layer.attn.Wo]
            if isinstance(layer.mlp, MLP):
                nn.init.uniform_(layer.mlp.Wi.weight, -bound, bound)
                nn.init.zeros_(layer.mlp.Wo.weight)
                lins += [layer.mlp.Wi, layer.mlp.Wo]
            for lin in lins:
                if lin.bias is not None:
                    nn.init.zeros_(lin.bias)
        nn.init.uniform_(self.head.dense.weight, -bound, bound)
        if self.head.dense.bias is not None:
            nn.init.zeros_(self.head.dense.bias)
        nn.init.normal_(self.decoder.weight, 0.0, emb_std if cfg.tie_word_embeddings else 0.001)
        if self.decoder.bias is not None:
            nn.init.zeros_(self.decoder.bias)

    def get_input_embeddings(self):
        return self.model.embeddings.tok_embeddings

    def get_output_embeddings(self):
        return self.decoder

    def num_parameters(self, only_trainable: bool = True) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)

    # ------------------------------------------------------------------ forward
    def _flatten_inputs(self, input_ids, attention_mask, labels, cu_seqlens, position_ids):
        """Brings any accepted input convention to flat (ids, labels, cu_seqlens, position_ids)."""
        if input_ids.dim() == 1:
            if cu_seqlens is None:
                raise ValueError("flat input_ids need cu_seqlens")
            T = input_ids.shape[0]
            if position_ids is None:
                position_ids = position_ids_from_cu_seqlens(cu_seqlens, T, input_ids.device)
            return input_ids, labels, cu_seqlens, position_ids, None
        B, S = input_ids.shape
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        keep = attention_mask.reshape(-1).bool()
        indices = torch.nonzero(keep, as_tuple=False).flatten()
        flat_ids = input_ids.reshape(-1)[indices]
        flat_labels = labels.reshape(-1)[indices] if labels is not None else None
        if cu_seqlens is None:
            lens = attention_mask.sum(dim=-1, dtype=torch.int32)
            cu_seqlens = F.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))
        position_ids = position_ids_from_cu_seqlens(cu_seqlens, flat_ids.shape[0], input_ids.device)
        return flat_ids, flat_labels, cu_seqlens, position_ids, (indices, B, S)

    def forward(self, input_ids, attention_mask=None, labels=None, cu_seqlens=None, max_seqlen=None,
                position_ids=None, masked_idx=None, masked_labels=None, return_logits=None,
                num_real_tokens: Optional[int] = None):
        """num_real_tokens (a host integer, as the packing collator reports it): flat batches of the
        static format end in a padding tail that carries no label and attends to nothing real. With
        the count known on the host the tail is cut off before the first kernel (the kernels take
        the token count at run time, there is no compiled static shape to keep), rounded up to a
        whole 128-token tile. Loss and gradients are unchanged."""
        cfg = self.config
        ids, flat_labels, cu, pos, pad_info = self._flatten_inputs(
            input_ids, attention_mask, labels, cu_seqlens, position_ids)
        T = ids.shape[0]
        if num_real_tokens is not None and pad_info is None and return_logits is None:
            keep = min(T, (int(num_real_tokens) + 127) // 128 * 128)
            if 0 < keep < T:
                ids, pos = ids[:keep], pos[:keep]
                if flat_labels is not None:
                    flat_labels = flat_labels[:keep]
                cu = torch.clamp(cu, max=keep)
                T = keep
        if int(max_seqlen or 0) > cfg.max_position_embeddings:
            raise ValueError(f"Sequence length {max_seqlen} exceeds max_position_embeddings="
                             f"{cfg.max_position_embeddings}")
        ctx = BatchContext(cu.to(ids.device), pos.to(ids.device), T)
        x, aux = self.model.forward_hidden(ids, ctx)

        if flat_labels is None and masked_labels is None:
            logits = self.decoder_logits(self.head(self.model.final_norm(x)))
            if pad_info is not None:
                indices, B, S = pad_info
                full = torch.zeros((B * S, logits.shape[-1]), dtype=logits.dtype, device=logits.device)
                full[indices] = logits
                logits = full.view(B, S, -1)
            return {"loss": None, "logits": logits}

        # the head only sees positions that carry a label: same loss, a fraction of the work
        if masked_idx is None:
            masked_idx = torch.nonzero(flat_labels != cfg.sparse_pred_ignore_index,
                                       as_tuple=False).flatten().to(torch.int32)
            masked_labels = flat_labels[masked_idx.long()]
        want_logits = bool(return_logits)
        if masked_idx.numel() == 0:
            loss = x.float().sum() * 0.0
            logits = None
        else:
            xm = ops.gather_rows(x, masked_idx)
            hm = self.head(self.model.final_norm(xm))
            loss, logits = ops.mlm_cross_entropy(hm, self.decoder.weight, self.decoder.bias,
                                                 masked_labels, want_logits)
        if want_logits and not cfg.sparse_prediction:
            # asked for logits next to the loss: every position, in the input's layout, as the
            # reference returns them (modeling.py:659-669, 713-725); with `sparse_prediction` only
            # the rows that carry a label (modeling.py:707-711). Training never asks.
            with torch.no_grad():
                logits = self.decoder_logits(self.head(self.model.final_norm(x)))
            if pad_info is not None:
                indices, B, S = pad_info
                full = torch.zeros((B * S, logits.shape[-1]), dtype=logits.dtype, device=logits.device)
                full[indices] = logits
                logits = full.view(B, S, -1)
        if aux is not None:
            loss = loss + cfg.moe.aux_loss_coef * aux
        return {"loss": loss, "logits": logits, "aux_loss": aux}

    def decoder_logits(self, h):
        return F.linear(h, self.decoder.weight, self.decoder.bias)


def estimate_flops_per_token(cfg: ModelConfig, seq_len: int) -> int:
    """Training FLOPs per token, the reference's formula (pure_pipeline.py:86-104):
    3 * (L * (8 h^2 + 4 s h + 6 h I) + 2 V h)."""
    h, I = cfg.hidden_size, cfg.intermediate_size
    per_layer = 8 * h * h + 4 * seq_len * h + 6 * h * I
    return 3 * (cfg.num_hidden_layers * per_layer + 2 * cfg.vocab_size * h)
