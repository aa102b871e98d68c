"""Optimizer engine for models whose MoE experts are split over data-parallel ranks
(`pretraining.expert_parallel_size` ranks per expert-parallel group; the world may hold several groups).

Dense parameters (attention, dense MLPs, routers, norms, embeddings) go through the sharded
data-parallel engine unchanged: gradients are summed over ranks, AdamW runs on the owned slice,
the bf16 copy is all-gathered (NCCL, or with `fused_comm` the peer-memory kernels with the
reduce-scatter under the backward pass). Expert weights are rank-local: every rank owns
num_experts / world experts, their gradients already contain the contributions of ALL ranks'
tokens (the rows travelled to the owner in the forward pass and their gradients came back in the
backward pass), so they are neither reduced nor gathered; they only share the scaling
1 / (grad_accum * world) and the global clipping norm with the dense part.

With `expert_parallel_size` < world the ranks form world / size expert-parallel groups of consecutive
ranks (rows travel inside a group only); the ranks with the same position in their groups hold the
same experts, and the gradients of those replicas are summed over that "expert data-parallel" group
before the update (`make_expert_groups`). Not tested on a GPU with more groups than one (it needs
four GPUs); the gloo test runs it on four CPU ranks.

The reference has neither MoE layers nor expert parallelism.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from nanoplm_b200.parallel.engine import ALIGN, AdamWHyper, ParamSlot, ShardedEngine, _round_up

EXPERT_PARAM_MARKERS = ("experts_Wi", "experts_Wo")


def is_expert_param(name: str) -> bool:
    return any(name.endswith(m) for m in EXPERT_PARAM_MARKERS)


def shard_model_experts(model: torch.nn.Module, group) -> int:
    """Splits the experts of every MoE layer of `model` over the ranks of `group` (in place).
    Returns the number of MoE layers touched."""
    from nanoplm_b200.models.moe import MoEMLP
    n = 0
    for m in model.modules():
        if isinstance(m, MoEMLP):
            m.shard_experts(group)
            n += 1
    return n


def make_expert_groups(ep_size: int):
    """(expert-parallel group, expert data-parallel group) of this rank for groups of `ep_size`
    consecutive ranks; (WORLD, None) when one group spans the world. Collective: every rank creates
    every group, in the same order."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if ep_size == world:
        return dist.group.WORLD, None
    if ep_size < 1 or world % ep_size:
        raise ValueError(f"expert_parallel_size ({ep_size}) must divide the number of ranks ({world})")
    ep_group = edp_group = None
    for g in range(world // ep_size):
        grp = dist.new_group(list(range(g * ep_size, (g + 1) * ep_size)))
        if rank // ep_size == g:
            ep_group = grp
    for k in range(ep_size):
        grp = dist.new_group(list(range(k, world, ep_size)))
        if rank % ep_size == k:
            edp_group = grp
    return ep_group, edp_group


class ExpertParallelEngine(ShardedEngine):
    def __init__(self, model, hyper: AdamWHyper, device, process_group=None,
                 compute_dtype: torch.dtype = torch.bfloat16, fused_comm: bool = False,
                 ep_group=None, edp_group=None):
        """ep_group: the ranks the experts are split over (default: all ranks of process_group);
        edp_group: the ranks holding the same experts as this one in other expert-parallel groups."""
        expert_names = [n for n, _ in model.named_parameters() if is_expert_param(n)]
        if not expert_names:
            raise ValueError("the model has no expert parameters (model.moe is not configured)")
        # dense part: the sharded engine, with the peer-memory optimizer step when asked for
        super().__init__(model, hyper, device, process_group, compute_dtype=compute_dtype, fused_comm=fused_comm,
                         exclude=expert_names)
        named = dict(model.named_parameters())
        self.x_slots: list[ParamSlot] = []
        off = 0
        for n in expert_names:
            p = named[n]
            self.x_slots.append(ParamSlot(n, p, off, p.numel(), p.shape, True))
            off = _round_up(off + p.numel(), ALIGN)
        self.x_total = max(off, ALIGN)
        dev = self.device
        self.x_params = torch.zeros(self.x_total, dtype=self.compute_dtype, device=dev)
        self.x_grad = torch.zeros(self.x_total, dtype=torch.float32, device=dev)
        self.x_master = torch.zeros(self.x_total, dtype=torch.float32, device=dev)
        self.x_exp_avg = torch.zeros(self.x_total, dtype=torch.float32, device=dev)
        self.x_exp_avg_sq = torch.zeros(self.x_total, dtype=torch.float32, device=dev)
        self._x_sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.ep_group = ep_group if ep_group is not None else self.pg
        self.edp_group = edp_group
        self.ep_world = dist.get_world_size(self.ep_group) if self.distributed else 1
        self.ep_rank = dist.get_rank(self.ep_group) if self.distributed else 0
        for s in self.x_slots:
            self.x_master[s.offset:s.offset + s.numel] = s.param.detach().to(dev, torch.float32).reshape(-1)
        if self.edp_group is not None:     # the replicas of an expert start from the same values
            dist.broadcast(self.x_master, src=dist.get_global_rank(self.edp_group, 0), group=self.edp_group)
        self.x_params.copy_(self.x_master.to(self.compute_dtype))
        self._rebind_experts()

    def _rebind_experts(self) -> None:
        for s in self.x_slots:
            s.param.data = self.x_params[s.offset:s.offset + s.numel].view(s.shape)
            s.param.grad = None
            if self.on_cuda:
                s.param.main_grad = self.x_grad[s.offset:s.offset + s.numel].view(s.shape)

    def num_parameters(self) -> int:
        return super().num_parameters() + self.ep_world * sum(s.numel for s in self.x_slots)

    def collect_autograd_grads(self) -> None:
        super().collect_autograd_grads()
        for s in self.x_slots:
            g = s.param.grad
            if g is not None:
                self.x_grad[s.offset:s.offset + s.numel].add_(g.reshape(-1).float())
                s.param.grad = None

    def zero_grad(self) -> None:
        super().zero_grad()
        self.x_grad.zero_()
        for s in self.x_slots:
            s.param.grad = None

    def step(self, lr: float, grad_accum: int = 1, extra_sumsq=None) -> torch.Tensor:
        self.collect_autograd_grads()
        if self.edp_group is not None:     # the other expert-parallel groups saw other tokens
            dist.all_reduce(self.x_grad, op=dist.ReduceOp.SUM, group=self.edp_group)
        # squared norm of all experts' gradients: the ranks of ONE expert-parallel group hold every expert once
        self._x_sumsq.zero_()
        if self.on_cuda:
            from nanoplm_b200.ops import kernels as K
            K.sumsq_(self.x_grad, self._x_sumsq)
        else:
            self._x_sumsq += self.x_grad.double().pow(2).sum().float()
        if self.distributed:
            dist.all_reduce(self._x_sumsq, op=dist.ReduceOp.SUM, group=self.ep_group)
        norm = super().step(lr, grad_accum, extra_sumsq=self._x_sumsq)   # leaves the global norm in _sumsq
        grad_scale = 1.0 / (grad_accum * self.world)
        if self.kernel_opt:
            from nanoplm_b200.ops import kernels as K
            K.adamw_(self.x_master, self.x_exp_avg, self.x_exp_avg_sq, self.x_grad, self.x_params,
                     self._hyper_dev[0], self._sumsq, zero_grad=False)
        else:
            self._adamw_cpu(self.x_master, self.x_exp_avg, self.x_exp_avg_sq, self.x_grad, self.x_params, 0, lr,
                            grad_scale)
        self.x_grad.zero_()
        return norm

    # ---- checkpoint: experts are gathered along their first axis ---------------------------------
    def _gather_experts(self, flat: torch.Tensor) -> dict:
        """name -> full tensor [num_experts, ...] (fp32, CPU); collective on every rank."""
        out = {}
        for s in self.x_slots:
            local = flat[s.offset:s.offset + s.numel].view(s.shape).contiguous()
            if self.distributed:
                parts = [torch.empty_like(local) for _ in range(self.ep_world)]
                dist.all_gather(parts, local, group=self.ep_group)
                local = torch.cat(parts, dim=0)
            out[s.name] = local.float().cpu()
        return out

    def _scatter_experts(self, flat: torch.Tensor, tensors: dict, strict: bool) -> None:
        for s in self.x_slots:
            t = tensors.get(s.name)
            if t is None:
                if strict:
                    raise KeyError(f"missing expert tensor in checkpoint: {s.name}")
                continue
            L = s.shape[0]
            mine = t[self.ep_rank * L:(self.ep_rank + 1) * L]
            if tuple(mine.shape) != tuple(s.shape):
                raise ValueError(f"{s.name}: checkpoint holds {tuple(t.shape)}, this rank needs {tuple(s.shape)} "
                                 f"x {self.ep_world} ranks")
            flat[s.offset:s.offset + s.numel] = mine.to(flat.device, torch.float32).reshape(-1)

    def full_state_dict_model(self, extra_tied=None) -> dict:
        sd = super().full_state_dict_model(extra_tied)
        sd.update(self._gather_experts(self.x_master))
        return sd

    def load_model_state_dict(self, sd: dict, strict: bool = True) -> None:
        sd = {k[len("_orig_mod."):] if k.startswith("_orig_mod.") else k: v for k, v in sd.items()}
        expert = {k: v for k, v in sd.items() if is_expert_param(k)}
        super().load_model_state_dict({k: v for k, v in sd.items() if k not in expert}, strict)
        self._scatter_experts(self.x_master, expert, strict)
        self.x_params.copy_(self.x_master.to(self.compute_dtype))
        self._rebind_experts()

    def optimizer_state_dict(self) -> dict:
        sd = super().optimizer_state_dict()
        sd["expert_parallel"] = {"exp_avg": self._gather_experts(self.x_exp_avg),
                                 "exp_avg_sq": self._gather_experts(self.x_exp_avg_sq)}
        return sd

    def load_optimizer_state_dict(self, sd: dict) -> None:
        super().load_optimizer_state_dict(sd)
        extra = sd.get("expert_parallel")
        if extra:
            self._scatter_experts(self.x_exp_avg, extra["exp_avg"], strict=False)
            self._scatter_experts(self.x_exp_avg_sq, extra["exp_avg_sq"], strict=False)

    def shard_state(self) -> dict:
        st = super().shard_state()
        st["experts"] = {"master": self.x_master.cpu(), "exp_avg": self.x_exp_avg.cpu(),
                         "exp_avg_sq": self.x_exp_avg_sq.cpu()}
        return st

    def load_shard_state(self, st: dict) -> None:
        super().load_shard_state(st)
        ex = st.get("experts")
        if ex:
            self.x_master.copy_(ex["master"])
            self.x_exp_avg.copy_(ex["exp_avg"])
            self.x_exp_avg_sq.copy_(ex["exp_avg_sq"])
            self.x_params.copy_(self.x_master.to(self.compute_dtype))
