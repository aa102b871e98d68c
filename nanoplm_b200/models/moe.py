"""Mixture-of-experts MLP: softmax router, top-k experts per token with renormalised gates, SwiGLU
experts, Switch-style load-balancing loss  aux = E * sum_e f_e * P_e  (f_e: share of assignments
routed to expert e, P_e: mean router probability of e).

On a GPU the whole layer runs through nanoplm_b200.ops.moe without a host synchronisation: router
top-k kernel, device-side plan (expert segments padded to 128-row tiles), token rows pushed into an
expert-major buffer, two grouped tcgen05 GEMMs over all experts in one launch each (SwiGLU fused
into the up-projection epilogue), and a gate-weighted pull. With expert parallelism (`ep_group`)
the experts are split over the ranks of the group and the rows travel over NVLink peer memory
inside the same push / pull kernels. Set `device_path=False` (or run on the CPU) for the plain
PyTorch restatement, which with `ep_group` uses an all-to-all (nanoplm_b200.parallel.expert) and
serves as the oracle and the collective-library baseline.

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
    def __init__(self, cfg: ModelConfig, ep_group=None, device_path: bool = True):
        super().__init__()
        self.device_path = device_path
        self._comm = None
        m = cfg.moe
        self.num_experts, self.top_k = m.num_experts, m.top_k
        self.inter = m.expert_intermediate_size
        self.capacity_factor = float(m.capacity_factor or 0.0)
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

    def shard_experts(self, group) -> None:
        """Keeps only this rank's experts (num_experts / world of them, a contiguous block) and routes
        the others' rows to their owners. Every rank must call this with identically initialised
        weights; the optimizer must treat the expert weights as rank-local
        (nanoplm_b200.parallel.expert_engine)."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if self.num_experts % world:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        if self.ep_world != 1:
            raise RuntimeError("experts are already sharded")
        L = self.num_experts // world
        self.ep_group, self.ep_world, self.ep_rank, self.local_experts = group, world, rank, L
        self.experts_Wi = nn.Parameter(self.experts_Wi.data[rank * L:(rank + 1) * L].clone())
        self.experts_Wo = nn.Parameter(self.experts_Wo.data[rank * L:(rank + 1) * L].clone())
        self._comm = None

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

    def _use_device_path(self, x: torch.Tensor) -> bool:
        return (self.device_path and x.is_cuda and x.dtype == torch.bfloat16 and self.hidden % 64 == 0
                and self.inter % 64 == 0 and self.num_experts <= 256 and self.top_k <= 8)

    def dropped_rows(self) -> int:
        """Expert rows this layer dropped so far because a rank's buffers were full (0 without expert
        parallelism, where the buffers are sized for the batch)."""
        return 0 if self._comm is None else self._comm.dropped_rows()

    def forward(self, x: torch.Tensor):
        T, C = x.shape
        if self._use_device_path(x):
            from nanoplm_b200.ops import moe as M
            if self._comm is None:
                self._comm = M.MoEComm(self.hidden, self.num_experts, self.top_k, group=self.ep_group,
                                       capacity_factor=self.capacity_factor)
            logits = ops.linear(x, self.router.weight)
            return M.moe_mlp(x, logits, self.experts_Wi, self.experts_Wo, self.top_k, self._comm)
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
