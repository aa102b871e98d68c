"""T5-style encoder teacher (ProtT5-XL shape by default: 24 layers, d_model 1024, 32 heads of 128,
d_ff 16384, ReLU feed-forward, RMS layer norms, relative-position bias with 32 buckets shared by all
layers, no attention scaling). Inference only.

Module / parameter names equal HF `T5EncoderModel` (`shared`, `encoder.block.N.layer.0.SelfAttention.
{q,k,v,o}`, `...relative_attention_bias`, `layer.1.DenseReluDense.{wi,wo}`, `layer_norm`,
`encoder.final_layer_norm`), so `Rostlab/prot_t5_xl_uniref50` weights load with `load_state_dict`;
benchmarks and offline machines use `random_init=True`. The reference wraps HF's implementation and
torch.compile (src/nanoplm/distillation/models/teacher/prott5.py:14-70); here the linear layers run
on the tcgen05 GEMM (ReLU and residual adds fused where the epilogue allows) and the norms on the
RMSNorm kernel. The bias-added attention uses PyTorch SDPA (a library call).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanoplm_b200.config.schema import TeacherConfig
from nanoplm_b200.data.tokenizer import TeacherTokenizer
from nanoplm_b200.ops import functional as ops


class _Lin(nn.Module):
    def __init__(self, i, o):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i))

    def forward(self, x, residual=None):
        return ops.linear(x, self.weight, None, residual=residual)


class _T5Norm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return ops.norm(x, self.weight, self.eps, rms=True)


def relative_position_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional T5 bucketing of relative positions (key - query)."""
    nb = num_buckets // 2
    ret = (rel > 0).long() * nb
    n = rel.abs()
    max_exact = nb // 2
    is_small = n < max_exact
    large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return ret + torch.where(is_small, n, large)


class SelfAttention(nn.Module):
    def __init__(self, cfg: TeacherConfig, has_bias: bool):
        super().__init__()
        inner = cfg.num_heads * cfg.d_kv
        self.h, self.dk = cfg.num_heads, cfg.d_kv
        self.q, self.k, self.v = _Lin(cfg.d_model, inner), _Lin(cfg.d_model, inner), _Lin(cfg.d_model, inner)
        self.o = _Lin(inner, cfg.d_model)
        self.cfg = cfg
        if has_bias:
            self.relative_attention_bias = nn.Embedding(cfg.relative_attention_num_buckets, cfg.num_heads)

    def compute_bias(self, S: int, device) -> torch.Tensor:
        pos = torch.arange(S, device=device)
        buckets = relative_position_bucket(pos[None, :] - pos[:, None], self.cfg.relative_attention_num_buckets,
                                           self.cfg.relative_attention_max_distance)
        return self.relative_attention_bias(buckets).permute(2, 0, 1)[None]     # [1, H, S, S]

    def compute_bias_table(self, S: int, device) -> torch.Tensor:
        """fp32 [H, 2S-1]: bias of relative position (key - query) = index - (S - 1)."""
        rel = torch.arange(-(S - 1), S, device=device)
        buckets = relative_position_bucket(rel, self.cfg.relative_attention_num_buckets,
                                           self.cfg.relative_attention_max_distance)
        return self.relative_attention_bias(buckets).float().t().contiguous()

    def _fused_qkv_weight(self) -> torch.Tensor:
        """[3*H*dk, d_model] = [Wq; Wk; Wv] (the teacher is frozen, so the copy is built once)."""
        w = getattr(self, "_wqkv", None)
        if w is None or w.device != self.q.weight.device or w.dtype != self.q.weight.dtype:
            w = torch.cat([self.q.weight, self.k.weight, self.v.weight], dim=0).detach().contiguous()
            self._wqkv = w
        return w

    def forward_native(self, x, fast, residual):
        """tcgen05 path: one fused QKV GEMM, attention with the relative-position bias table in the
        kernel (nanoplm_b200/csrc/attention_bias.cu), output projection with the residual add."""
        from nanoplm_b200.ops import kernels as K
        B, S, _ = x.shape
        x2 = x.reshape(B * S, -1)
        qkv = ops.linear(x2, self._fused_qkv_weight())
        y = K.fa_bias_fwd(qkv, fast["seq_start"], fast["seq_end"], fast["table"], self.h, self.dk, 1.0)
        return self.o(y, residual=residual.reshape(B * S, -1)).view(B, S, -1)

    def forward(self, x, bias, residual):
        if isinstance(bias, dict):
            return self.forward_native(x, bias, residual)
        B, S, _ = x.shape
        x2 = x.reshape(B * S, -1)
        q = self.q(x2).view(B, S, self.h, self.dk).transpose(1, 2)
        k = self.k(x2).view(B, S, self.h, self.dk).transpose(1, 2)
        v = self.v(x2).view(B, S, self.h, self.dk).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype), scale=1.0)
        y = y.transpose(1, 2).reshape(B * S, self.h * self.dk)
        return self.o(y, residual=residual.reshape(B * S, -1)).view(B, S, -1)


class _AttnLayer(nn.Module):
    def __init__(self, cfg, has_bias):
        super().__init__()
        self.SelfAttention = SelfAttention(cfg, has_bias)
        self.layer_norm = _T5Norm(cfg.d_model, cfg.layer_norm_epsilon)

    def forward(self, x, bias):
        return self.SelfAttention(self.layer_norm(x), bias, residual=x)


class _DenseReluDense(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.wi, self.wo = _Lin(cfg.d_model, cfg.d_ff), _Lin(cfg.d_ff, cfg.d_model)

    def forward(self, x2, residual):
        return self.wo(ops.linear(x2, self.wi.weight, act="relu"), residual=residual)   # ReLU in the GEMM epilogue


class _FFLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.DenseReluDense = _DenseReluDense(cfg)
        self.layer_norm = _T5Norm(cfg.d_model, cfg.layer_norm_epsilon)

    def forward(self, x):
        B, S, C = x.shape
        return self.DenseReluDense(self.layer_norm(x).reshape(B * S, C), x.reshape(B * S, C)).view(B, S, C)


class _Block(nn.Module):
    def __init__(self, cfg, has_bias):
        super().__init__()
        self.layer = nn.ModuleList([_AttnLayer(cfg, has_bias), _FFLayer(cfg)])

    def forward(self, x, bias):
        return self.layer[1](self.layer[0](x, bias))


class _Stack(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.block = nn.ModuleList([_Block(cfg, i == 0) for i in range(cfg.num_layers)])
        self.final_layer_norm = _T5Norm(cfg.d_model, cfg.layer_norm_epsilon)


class T5EncoderTeacher(nn.Module):
    def __init__(self, cfg: Optional[TeacherConfig] = None, random_init: bool = True, seed: int = 0):
        super().__init__()
        self.cfg = cfg or TeacherConfig()
        self.tokenizer = TeacherTokenizer(self.cfg.vocab_size)
        self.shared = nn.Embedding(self.cfg.vocab_size, self.cfg.d_model)
        self.encoder = _Stack(self.cfg)
        if random_init:
            g = torch.Generator().manual_seed(seed)
            with torch.no_grad():
                for name, p in self.named_parameters():
                    if p.ndim >= 2:
                        p.copy_(torch.randn(p.shape, generator=g) * (p.shape[-1] ** -0.5))
        for p in self.parameters():
            p.requires_grad_(False)
        self.native_attention = True   # False: PyTorch SDPA with a dense bias (the restatement)
        self.eval()

    @classmethod
    def from_pretrained(cls, name_or_path: str, cfg: Optional[TeacherConfig] = None) -> "T5EncoderTeacher":
        """Loads HF T5EncoderModel weights (needs the files locally or network access)."""
        from transformers import T5EncoderModel
        hf = T5EncoderModel.from_pretrained(name_or_path)
        c = hf.config
        cfg = cfg or TeacherConfig(vocab_size=c.vocab_size, d_model=c.d_model, d_kv=c.d_kv, d_ff=c.d_ff,
                                   num_layers=c.num_layers, num_heads=c.num_heads,
                                   relative_attention_num_buckets=c.relative_attention_num_buckets,
                                   relative_attention_max_distance=c.relative_attention_max_distance,
                                   layer_norm_epsilon=c.layer_norm_epsilon, name=name_or_path)
        m = cls(cfg, random_init=False)
        sd = {k: v for k, v in hf.state_dict().items() if k != "encoder.embed_tokens.weight"}
        m.load_state_dict(sd, strict=True)
        return m

    @staticmethod
    def preprocess(seq: str) -> str:
        return TeacherTokenizer.preprocess(seq)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                lengths: Optional[list] = None) -> torch.Tensor:
        """(B, S) token ids -> (B, S, d_model) last hidden state.

        lengths: number of real (left-aligned) tokens of every row as host integers. When given on
        the native path, the padding is removed before the first layer (the whole encoder then
        runs on the real tokens only, like the student's varlen path) and the output is scattered
        back into the padded layout with zeros at the padding positions. Without it the padded
        batch is processed as is, padding tokens attending to themselves."""
        B, S = input_ids.shape
        attn0 = self.encoder.block[0].layer[0].SelfAttention
        native = (input_ids.is_cuda and self.shared.weight.dtype == torch.bfloat16 and self.cfg.d_kv in (64, 128)
                  and S <= 2048 and self.native_attention)
        if native and lengths is not None:
            dev = input_ids.device
            lens = [int(min(max(n, 0), S)) for n in lengths]
            idx_host = torch.cat([torch.arange(n, dtype=torch.int64) + b * S for b, n in enumerate(lens)])
            cu_host = torch.zeros(B + 1, dtype=torch.int32)
            cu_host[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int32), 0)
            idx = idx_host.pin_memory().to(dev, non_blocking=True)
            cu = cu_host.pin_memory().to(dev, non_blocking=True)
            T = int(idx_host.numel())
            x = self.shared(input_ids.reshape(-1)[idx]).unsqueeze(0)                  # [1, T, d]
            start, end = ops.seq_bounds(cu, T)
            fast = {"seq_start": start, "seq_end": end, "table": attn0.compute_bias_table(max(lens + [1]), dev)}
            for blk in self.encoder.block:
                x = blk(x, fast)
            y = self.encoder.final_layer_norm(x)[0]
            out = torch.zeros((B * S, y.shape[-1]), dtype=y.dtype, device=dev)
            out.index_copy_(0, idx, y)
            return out.view(B, S, -1)
        x = self.shared(input_ids)
        if native:
            # key range of every token of the padded batch: its sequence's valid prefix; padding
            # tokens see themselves only (their outputs are never used)
            dev = x.device
            if attention_mask is None:
                lengths_t = torch.full((B,), S, device=dev, dtype=torch.int32)
            else:
                lengths_t = attention_mask.sum(dim=1).to(torch.int32)
            pos = torch.arange(S, device=dev, dtype=torch.int32)[None, :]
            base = (torch.arange(B, device=dev, dtype=torch.int32) * S)[:, None]
            valid = pos < lengths_t[:, None]
            start = torch.where(valid, base.expand(B, S), base + pos)
            end = torch.where(valid, (base + lengths_t[:, None]).expand(B, S), base + pos + 1)
            fast = {"seq_start": start.reshape(-1).contiguous(), "seq_end": end.reshape(-1).contiguous(),
                    "table": attn0.compute_bias_table(S, dev)}
            for blk in self.encoder.block:
                x = blk(x, fast)
            return self.encoder.final_layer_norm(x)
        bias = attn0.compute_bias(S, input_ids.device)
        if attention_mask is not None:
            neg = torch.finfo(torch.float32).min
            bias = bias.float() + (1.0 - attention_mask[:, None, None, :].float()) * neg
        for blk in self.encoder.block:
            x = blk(x, bias)
        return self.encoder.final_layer_norm(x)


class BaseTeacher:
    """What the distillation code needs from a teacher (reference: teacher/base.py:9-29): a
    tokenizer, an encoder module whose forward gives the last hidden state, and the text
    preprocessing that goes before tokenisation."""

    def __init__(self, device: Optional[str] = None) -> None:
        self.device = str(device) if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")

    @property
    def tokenizer(self):
        raise NotImplementedError

    @property
    def encoder_model(self) -> nn.Module:
        raise NotImplementedError

    def preprocess(self, sequence: str) -> str:
        raise NotImplementedError


class ProtT5(BaseTeacher):
    """The ProtT5-XL encoder as a teacher (reference: teacher/prott5.py:14-70). `model_name` is a hub
    id or a local directory with the HF files; `random_init=True` builds the same architecture with
    seeded random weights (benchmarks, machines without the weights). The encoder is created on
    first use and cached; on CUDA it runs in bf16 on this package's kernels, no compiler step."""

    def __init__(self, model_name: str = "Rostlab/prot_t5_xl_uniref50", device: Optional[str] = None,
                 random_init: bool = False, cfg: Optional[TeacherConfig] = None, seed: int = 0):
        super().__init__(device)
        self.model_name, self.random_init, self.cfg, self.seed = model_name, random_init, cfg, seed
        self._encoder_model: Optional[T5EncoderTeacher] = None
        self._tokenizer: Optional[TeacherTokenizer] = None

    @property
    def encoder_model(self) -> T5EncoderTeacher:
        if self._encoder_model is None:
            if self.random_init:
                m = T5EncoderTeacher(self.cfg, random_init=True, seed=self.seed)
            else:
                m = T5EncoderTeacher.from_pretrained(self.model_name, self.cfg)
            m = m.to(self.device)
            if "cuda" in self.device:
                m = m.to(torch.bfloat16)
            self._encoder_model = m.eval()
        return self._encoder_model

    @property
    def tokenizer(self) -> TeacherTokenizer:
        if self._tokenizer is None:
            self._tokenizer = TeacherTokenizer((self.cfg or TeacherConfig()).vocab_size)
        return self._tokenizer

    def get_layer_weights(self) -> dict:
        return {k: v.detach() for k, v in self.encoder_model.state_dict().items()}

    def get_layer_by_name(self, layer_name: str) -> torch.Tensor:
        sd = self.get_layer_weights()
        if layer_name not in sd:
            raise ValueError(f"Layer {layer_name} not found in model.")
        return sd[layer_name]

    def preprocess(self, sequence: str) -> str:
        return TeacherTokenizer.preprocess(sequence or "")

    @torch.no_grad()
    def embed(self, sequences: list[str], max_length: Optional[int] = None) -> tuple[torch.Tensor, torch.Tensor]:
        """(B, S, d_model) last hidden states and the (B, S) attention mask of raw sequences."""
        enc = self.tokenizer([self.preprocess(s) for s in sequences],
                             padding="max_length" if max_length else True, max_length=max_length,
                             truncation=bool(max_length), return_tensors="pt")
        ids, mask = enc["input_ids"].to(self.device), enc["attention_mask"].to(self.device)
        out = self.encoder_model(ids, mask, lengths=mask.sum(dim=1).tolist())
        return out, mask
