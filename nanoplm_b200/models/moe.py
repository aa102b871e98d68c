"""Mixture-of-experts MLP: softmax router, top-k experts per token with renormalised gates, SwiGLU
experts, Switch-style load-balancing loss  aux = E * sum_e f_e * P_e  (f_e: share of assignments
routed to expert e, P_e: mean router probability of e).

Tokens are sorted by expert once per layer (a permutation of T*k rows), every expert runs its two
GEMMs on a contiguous row slice with the tcgen05 GEMM (SwiGLU fused into the up-projection
epilogue), and the outputs are combined with the gate weights. With expert parallelism
(`ep_group`) the experts are split over the ranks of the group and the permuted rows travel through
an all-to-all before and after the expert GEMMs (nanoplm_b200.parallel.expert).

The reference has no MoE layers.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from nanoplm_b200.config.schema import ModelConfig
from nanoplm_b200.ops import functional as ops
from nanoplm_b200.ops.functional import _has_main_grad


def route_topk(logits: torch.Tensor, top_k: int):
    """Returns (gates [T,k] renormalised, experts [T,k] int64, aux loss scalar)."""
    probs = torch.softmax(logits.float(), dim=-1)
    gates, experts = torch.topk(probs, top_k, dim=-1)
    gates = gates / gates.sum(dim=-1, keepdim=True).clamp(min=1e-9)
    E = logits.shape[-1]
    counts = torch.zeros(E, dtype=torch.float32, device=logits.device)
    counts.scatter_add_(0, experts.reshape(-1), torch.ones(experts.numel(), device=logits.device))
    f = counts / max(1, experts.numel())
    aux = E * (f * probs.mean(dim=0)).sum()
    return gates, experts, aux


def _expert_weight(param: torch.Tensor, e: int) -> torch.Tensor:
    w = param[e]
    if _has_main_grad(param):
        w.main_grad = param.main_grad[e]
    return w


class MoEMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, ep_group=None):
        super().__init__()
        m = cfg.moe
        self.num_experts, self.top_k = m.num_experts, m.top_k
        self.inter = m.expert_intermediate_size
        self.hidden = cfg.hidden_size
        self.ep_group = ep_group
        self.ep_world = 1
        self.ep_rank = 0
        if ep_group is not None:
            import torch.distributed as dist
            self.ep_world, self.ep_rank = dist.get_world_size(ep_group), dist.get_rank(ep_group)
        if self.num_experts % self.ep_world:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.local_experts = self.num_experts // self.ep_world
        self.router = nn.Linear(cfg.hidden_size, self.num_experts, bias=False)
        nn.init.normal_(self.router.weight, 0.0, 0.02)
        bound = math.sqrt(3.0 / cfg.hidden_size)
        self.experts_Wi = nn.Parameter(torch.empty(self.local_experts, 2 * self.inter, cfg.hidden_size).uniform_(-bound, bound))
        self.experts_Wo = nn.Parameter(torch.zeros(self.local_experts, cfg.hidden_size, self.inter))

    def _run_experts(self, rows: torch.Tensor, counts: list[int]) -> torch.Tensor:
        """rows sorted by local expert; counts[e] rows belong to local expert e."""
        out = torch.empty((rows.shape[0], self.hidden), dtype=rows.dtype, device=rows.device)
        pieces, start = [], 0
        for e, n in enumerate(counts):
            if n > 0:
                xs = rows[start:start + n]
                h = ops.linear(xs, _expert_weight(self.experts_Wi, e), act="swiglu")
                pieces.append(ops.linear(h, _expert_weight(self.experts_Wo, e)))
            start += n
        if not pieces:
            return out.zero_() + 0.0 * (self.experts_Wi.sum() + self.experts_Wo.sum()).to(out.dtype)
        return torch.cat(pieces, dim=0)

    def forward(self, x: torch.Tensor):
        T, C = x.shape
        logits = F.linear(x, self.router.weight)
        gates, experts, aux = route_topk(logits, self.top_k)
        flat_e = experts.reshape(-1)
        order = torch.argsort(flat_e, stable=True)                       # rows grouped by expert
        token_of = (order // self.top_k).to(torch.int32)
        counts = torch.bincount(flat_e, minlength=self.num_experts)
        rows = ops.gather_rows(x, token_of) if self.top_k == 1 else x[token_of.long()]
        if self.ep_group is None:
            y_rows = self._run_experts(rows, counts.tolist())
        else:
            from nanoplm_b200.parallel.expert import expert_parallel_apply
            y_rows = expert_parallel_apply(self, rows, counts)
        w = gates.reshape(-1)[order].to(y_rows.dtype)
        y = torch.zeros((T, C), dtype=y_rows.dtype, device=x.device)
        y.index_add_(0, token_of.long(), y_rows * w[:, None])
        return y, aux
