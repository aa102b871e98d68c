"""Sharded data-parallel engine: flat parameter storage, fp32 gradient accumulation, sharded AdamW.

What the reference gets from FSDP2 + torch.optim.AdamW + clip_grad_norm_
(src/nanoplm/pretraining/pure_pipeline.py:107-147, 479-506, 755-764) is organised differently here:

  * all parameters live in ONE flat bf16 buffer (the compute copy, complete on every rank — at
    169 M parameters that is 0.34 GB of 180 GB, so nothing is re-gathered per micro-step), laid out
    as [weight-decay tensors | no-decay tensors], every tensor starting on a 128-byte boundary so
    it can be a TMA operand in place;
  * gradients accumulate in one flat fp32 buffer (`main_grad`); weight-gradient GEMMs add into it
    from their epilogue, across micro-steps, so there is no separate accumulation pass;
  * the optimizer state (fp32 master weights, exp_avg, exp_avg_sq) is sharded: rank r owns the
    r-th contiguous slice of the flat index space;
  * `step()` = reduce-scatter(main_grad) -> global grad norm -> clip + AdamW on the owned slice ->
    all-gather of the updated bf16 slice. With `fused_comm` on a multi-GPU NVLink node the three
    stages run as one P2P kernel (nanoplm_b200.comm); otherwise NCCL (GPU) or gloo (CPU ranks).

Weight-decay grouping follows the reference (`_use_weight_decay`, pure_pipeline.py:68-76): no decay
for tensors with fewer than two dimensions or with "bias" / "norm" in their name.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

ALIGN = 64  # elements; 64 bf16 = 128 bytes


def use_weight_decay(name: str, p: torch.Tensor) -> bool:
    lname = name.lower()
    if not p.requires_grad or p.ndim < 2:
        return False
    return not ("bias" in lname or "norm" in lname)


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: torch.Size
    decay: bool


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class AdamWHyper:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0


def _invalidate_fp8_weights() -> None:
    """Quantised copies of the weights are valid for one optimizer step only."""
    import sys
    mod = sys.modules.get("nanoplm_b200.ops.fp8")
    if mod is not None:
        mod.invalidate_weight_cache()


class ShardedEngine:
    def __init__(self, model: nn.Module, hyper: AdamWHyper, device: torch.device,
                 process_group=None, compute_dtype: torch.dtype = torch.bfloat16,
                 fused_comm: bool = False, exclude: Iterable[str] = (), decay_all: bool = False):
        self.model = model
        self.hyper = hyper
        self.device = torch.device(device)
        self.pg = process_group
        self.distributed = dist.is_available() and dist.is_initialized() and (
            dist.get_world_size(process_group) > 1)
        self.world = dist.get_world_size(process_group) if self.distributed else 1
        self.rank = dist.get_rank(process_group) if self.distributed else 0
        self.on_cuda = self.device.type == "cuda"
        self.compute_dtype = compute_dtype if self.on_cuda else torch.float32
        # the optimizer kernels write the bf16 compute copy; an fp32 compute copy on a GPU
        # (`bf16: false`) takes the PyTorch restatement of the update instead
        self.kernel_opt = self.on_cuda and self.compute_dtype == torch.bfloat16
        self.step_count = 0
        self.fused = None
        tied = getattr(model, "_tied_weights_keys", {}) or {}
        self._shared_names = set(tied.values()) | set(tied.keys())

        # ---- flat layout ------------------------------------------------------------------
        seen: dict[int, str] = {}
        named = []
        exclude = tuple(exclude)
        for name, p in model.named_parameters():
            if not p.requires_grad or id(p) in seen or any(name.startswith(e) for e in exclude):
                continue
            seen[id(p)] = name
            named.append((name, p))
        # decay_all: one group with the weight decay on every tensor, norms and biases included, which
        # is what `AdamW(model.parameters())` does (reference: distillation/pipeline.py:669)
        decay = [(n, p) for n, p in named if decay_all or use_weight_decay(n, p)]
        no_decay = [(n, p) for n, p in named if not (decay_all or use_weight_decay(n, p))]
        self.slots: list[ParamSlot] = []
        off = 0
        for group, flag in ((decay, True), (no_decay, False)):
            for n, p in group:
                self.slots.append(ParamSlot(n, p, off, p.numel(), p.shape, flag))
                off = _round_up(off + p.numel(), ALIGN)
            if flag:
                off = _round_up(off, ALIGN)
                self.decay_end = off
        if not decay:
            self.decay_end = 0
        self.total = _round_up(max(off, ALIGN), ALIGN * self.world)
        self._plan_ownership()

        dev = self.device
        sym = None
        if fused_comm and self.kernel_opt and self.distributed:
            from nanoplm_b200.comm.fused_optimizer import FusedShardedStep
            sym = FusedShardedStep.allocate(self.total, self.world, dev, self.pg, self.compute_dtype)
        if sym is not None:   # gradients and parameters live in peer-mapped memory
            self.main_grad, self.flat_params = sym[0].tensor, sym[1].tensor
        else:
            self.flat_params = torch.zeros(self.total, dtype=self.compute_dtype, device=dev)
            self.main_grad = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.master = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._hyper_dev = torch.zeros(2, 9, dtype=torch.float32, device=dev)
        self._hyper_host = torch.zeros(2, 9, dtype=torch.float32,
                                       pin_memory=self.on_cuda)

        full_master = torch.zeros(self.total, dtype=torch.float32, device=dev)
        for s in self.slots:
            src = s.param.detach().to(device=dev, dtype=torch.float32).reshape(-1)
            full_master[s.offset:s.offset + s.numel] = src
        if self.distributed:  # identical start on every rank (rank 0's initialisation wins)
            dist.broadcast(full_master, src=dist.get_global_rank(self.pg, 0) if self.pg else 0, group=self.pg)
        self.master.copy_(self._take_local(full_master))
        self.flat_params.copy_(full_master.to(self.compute_dtype))
        del full_master
        self._rebind()
        if sym is not None:
            self.fused = self._make_fused(sym)
            dist.barrier(group=self.pg)
        self._slot_of = {id(s.param): s for s in self.slots}

    # ---- who owns which part of the flat index space (overridden by ParamShardedEngine) ----------
    def _plan_ownership(self) -> None:
        """Rank r owns the r-th contiguous slice of the flat space; `shard` = elements of optimizer
        state this rank stores."""
        self.shard = self.total // self.world
        self.lo, self.hi = self.rank * self.shard, (self.rank + 1) * self.shard

    def _take_local(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's part of a full flat vector, in the layout of its optimizer state."""
        return full[self.lo:self.hi]

    def _make_fused(self, sym):
        from nanoplm_b200.comm.fused_optimizer import FusedShardedStep
        return FusedShardedStep(self, *sym)

    # ---- overlap of the gradient reduction with the backward pass --------------------------
    def begin_last_microstep(self) -> None:
        """Tells the engine that the micro-batch about to run is the last one of this optimizer
        step: with the fused communication path, every parameter's reduce-scatter then starts as
        soon as its weight-gradient kernel has been launched, under the rest of the backward pass.
        Must be called by every rank (the reductions contain peer barriers). No-op otherwise."""
        if self.fused is None:
            return
        from nanoplm_b200.ops import functional as ops
        self.fused.arm()
        ops.set_wgrad_ready_callback(self._on_wgrad_ready)

    def _on_wgrad_ready(self, param) -> None:
        s = self._slot_of.get(id(param))
        # tied / shared parameters receive several gradient contributions: they wait for the step
        if s is not None and s.name not in self._shared_names:
            self.fused.on_wgrad_ready((s.offset, s.offset + s.numel))

    # ---- parameter views ------------------------------------------------------------------
    def _rebind(self) -> None:
        """Points every parameter (and its main_grad) at its slice of the flat buffers."""
        for s in self.slots:
            s.param.data = self.flat_params[s.offset:s.offset + s.numel].view(s.shape)
            s.param.grad = None
            if self.on_cuda:
                s.param.main_grad = self.main_grad[s.offset:s.offset + s.numel].view(s.shape)
        # buffers and excluded parameters follow the device / dtype of the compute copy
        owned = {id(s.param) for s in self.slots}
        for p in self.model.parameters():
            if id(p) not in owned:
                p.data = p.data.to(device=self.device, dtype=self.compute_dtype if p.is_floating_point() else p.dtype)
        for b in self.model.buffers():
            b.data = b.data.to(self.device)

    def num_parameters(self) -> int:
        return sum(s.numel for s in self.slots)

    # ---- gradient handling ----------------------------------------------------------------
    def collect_autograd_grads(self) -> None:
        """Adds any `.grad` autograd produced (CPU path, or ops without a fused epilogue) into the
        flat fp32 buffer and frees it."""
        for s in self.slots:
            g = s.param.grad
            if g is not None:
                self.main_grad[s.offset:s.offset + s.numel].add_(g.reshape(-1).float())
                s.param.grad = None

    def zero_grad(self) -> None:
        self.main_grad.zero_()
        for s in self.slots:
            s.param.grad = None

    # ---- optimizer step -------------------------------------------------------------------
    def _fill_hyper(self, lr: float, grad_scale: float) -> None:
        h = self.hyper
        t = self.step_count
        bc1, bc2 = 1.0 - h.beta1 ** t, 1.0 - h.beta2 ** t
        for i, wd in enumerate((h.weight_decay, 0.0)):
            self._hyper_host[i] = torch.tensor(
                [lr, h.beta1, h.beta2, h.eps, wd, bc1, bc2, grad_scale, h.max_grad_norm])
        self._hyper_dev.copy_(self._hyper_host, non_blocking=True)

    def step(self, lr: float, grad_accum: int = 1, extra_sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One optimizer step. Returns the global gradient norm (a device scalar; no host sync).
        extra_sumsq: sum of squares of gradients held outside this engine's flat buffer (already
        summed over ranks, same scaling); it enters the clipping norm."""
        self.collect_autograd_grads()
        self.step_count += 1
        _invalidate_fp8_weights()
        grad_scale = 1.0 / (grad_accum * self.world)
        self._fill_hyper(lr, grad_scale)
        if self.fused is not None:
            from nanoplm_b200.ops import functional as ops
            ops.set_wgrad_ready_callback(None)
            return self.fused.step(lr, grad_scale, extra_sumsq)
        # 1. reduce-scatter: the owned slice of main_grad becomes the sum over ranks
        if self.distributed:
            shard_grad = torch.empty(self.shard, dtype=torch.float32, device=self.device)
            if self.on_cuda:
                dist.reduce_scatter_tensor(shard_grad, self.main_grad, op=dist.ReduceOp.SUM, group=self.pg)
            else:  # gloo has no reduce_scatter: all-reduce and slice
                dist.all_reduce(self.main_grad, op=dist.ReduceOp.SUM, group=self.pg)
                shard_grad.copy_(self.main_grad[self.lo:self.hi])
        else:
            shard_grad = self.main_grad
        # 2. global gradient norm of the scaled gradient
        self._sumsq.zero_()
        if self.on_cuda:
            from nanoplm_b200.ops import kernels as K
            K.sumsq_(shard_grad, self._sumsq)
        else:
            self._sumsq += shard_grad.double().pow(2).sum().float()
        if self.distributed:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=self.pg)
        if extra_sumsq is not None:
            self._sumsq += extra_sumsq.to(self._sumsq.dtype).reshape(1)
        grad_norm = self._sumsq.sqrt() * grad_scale
        # 3. clip + AdamW on the owned slice, decay part then no-decay part
        new_shard = self.flat_params[self.lo:self.hi]
        for i, (a, b) in enumerate(((0, self.decay_end), (self.decay_end, self.total))):
            a, b = max(a, self.lo), min(b, self.hi)
            if b <= a:
                continue
            sl = slice(a - self.lo, b - self.lo)
            if self.kernel_opt:
                from nanoplm_b200.ops import kernels as K
                K.adamw_(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], shard_grad[sl],
                         new_shard[sl], self._hyper_dev[i], self._sumsq, zero_grad=False)
            else:
                self._adamw_reference(sl, shard_grad, new_shard, i, lr, grad_scale)
        # 4. all-gather the updated compute copy
        if self.distributed:
            dist.all_gather_into_tensor(self.flat_params, new_shard.clone(), group=self.pg)
        self.main_grad.zero_()
        return grad_norm

    def _adamw_reference(self, sl, grad, out, group, lr, grad_scale) -> None:
        self._adamw_cpu(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], grad[sl], out[sl], group, lr,
                        grad_scale)

    def _adamw_cpu(self, p, m, v, grad, out, group, lr, grad_scale) -> None:
        """fp32 PyTorch restatement of the AdamW kernel (clip by the global norm in self._sumsq)."""
        h = self.hyper
        wd = h.weight_decay if group == 0 else 0.0
        norm = float(self._sumsq.sqrt()) * grad_scale
        scale = grad_scale
        if h.max_grad_norm > 0:
            scale *= min(1.0, h.max_grad_norm / (norm + 1e-6))
        g = grad * scale
        sl = slice(None)
        t = self.step_count
        p.mul_(1.0 - lr * wd)
        m.mul_(h.beta1).add_(g, alpha=1 - h.beta1)
        v.mul_(h.beta2).addcmul_(g, g, value=1 - h.beta2)
        denom = (v.sqrt() / math.sqrt(1 - h.beta2 ** t)).add_(h.eps)
        p.addcdiv_(m, denom, value=-lr / (1 - h.beta1 ** t))
        out[sl] = p.to(out.dtype)

    # ---- state (checkpoint) -----------------------------------------------------------------
    def _gather_full(self, shard: torch.Tensor) -> torch.Tensor:
        if not self.distributed:
            return shard
        full = torch.empty(self.total, dtype=shard.dtype, device=shard.device)
        if self.on_cuda:
            dist.all_gather_into_tensor(full, shard.contiguous(), group=self.pg)
        else:
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.contiguous(), group=self.pg)
            full = torch.cat(parts)
        return full

    def full_state_dict_model(self, extra_tied: Optional[dict] = None) -> dict:
        """fp32 model state dict with the module's own key names (collective on every rank)."""
        full = self._gather_full(self.master).cpu()
        by_id = {id(s.param): full[s.offset:s.offset + s.numel].view(s.shape).clone() for s in self.slots}
        sd = {}
        for key, t in self.model.state_dict(keep_vars=True).items():
            sd[key] = by_id[id(t)] if id(t) in by_id else t.detach().float().cpu()
        return sd

    def load_model_state_dict(self, sd: dict, strict: bool = True) -> None:
        sd = {k[len("_orig_mod."):] if k.startswith("_orig_mod.") else k: v for k, v in sd.items()}
        full = self._gather_full(self.master).clone()
        names = {s.name for s in self.slots}
        missing = []
        for s in self.slots:
            t = sd.get(s.name)
            if t is None:
                for alias, target in getattr(self.model, "_tied_weights_keys", {}).items():
                    if target == s.name and alias in sd:
                        t = sd[alias]
            if t is None:
                missing.append(s.name)
                continue
            full[s.offset:s.offset + s.numel] = t.to(device=full.device, dtype=torch.float32).reshape(-1)
        if strict and missing:
            raise KeyError(f"missing keys in checkpoint: {missing}")
        self.master.copy_(self._take_local(full))
        self.flat_params.copy_(full.to(self.compute_dtype))
        self._params_replaced()
        # non-flat entries (buffers) go through the module
        rest = {k: v for k, v in sd.items() if k not in names}
        own = self.model.state_dict(keep_vars=True)
        for k, v in rest.items():
            if k in own and own[k].shape == v.shape and id(own[k]) not in {id(s.param) for s in self.slots}:
                own[k].data.copy_(v.to(own[k].device, own[k].dtype))

    def optimizer_state_dict(self) -> dict:
        """torch.optim.AdamW-compatible state dict (full tensors; collective on every rank).
        Parameter order = decay group then no-decay group (reference: pure_pipeline.py:127-130)."""
        m = self._gather_full(self.exp_avg).cpu()
        v = self._gather_full(self.exp_avg_sq).cpu()
        h = self.hyper
        state, groups = {}, []
        idx = 0
        for flag, wd in ((True, h.weight_decay), (False, 0.0)):
            ids = []
            for s in self.slots:
                if s.decay != flag:
                    continue
                if self.step_count > 0:
                    state[idx] = {
                        "step": torch.tensor(float(self.step_count)),
                        "exp_avg": m[s.offset:s.offset + s.numel].view(s.shape).clone(),
                        "exp_avg_sq": v[s.offset:s.offset + s.numel].view(s.shape).clone(),
                    }
                ids.append(idx)
                idx += 1
            if not ids:
                continue                            # torch optimizers have no empty groups
            groups.append({"lr": h.lr, "betas": (h.beta1, h.beta2), "eps": h.eps, "weight_decay": wd,
                           "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                           "differentiable": False, "fused": None, "decoupled_weight_decay": True,
                           "params": ids})
        return {"state": state, "param_groups": groups}

    def load_optimizer_state_dict(self, sd: dict) -> None:
        m = self._gather_full(self.exp_avg).clone()
        v = self._gather_full(self.exp_avg_sq).clone()
        ordered = [s for s in self.slots if s.decay] + [s for s in self.slots if not s.decay]
        step = 0
        for idx, s in enumerate(ordered):
            st = sd["state"].get(idx) or sd["state"].get(str(idx))
            if st is None:
                continue
            m[s.offset:s.offset + s.numel] = st["exp_avg"].to(m.device, torch.float32).reshape(-1)
            v[s.offset:s.offset + s.numel] = st["exp_avg_sq"].to(v.device, torch.float32).reshape(-1)
            step = max(step, int(float(st["step"])))
        self.exp_avg.copy_(self._take_local(m))
        self.exp_avg_sq.copy_(self._take_local(v))
        self.step_count = step

    def shard_state(self) -> dict:
        """This rank's slice only (sharded checkpoint fast path)."""
        return {"rank": self.rank, "world": self.world, "total": self.total, "step": self.step_count,
                "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu()}

    def load_shard_state(self, st: dict) -> None:
        if st["world"] != self.world or st["total"] != self.total:
            raise ValueError("sharded checkpoint was written with a different world size / layout")
        self.master.copy_(st["master"])
        self.exp_avg.copy_(st["exp_avg"])
        self.exp_avg_sq.copy_(st["exp_avg_sq"])
        self.step_count = int(st["step"])
        full = self._gather_full(self.master)
        self.flat_params.copy_(full.to(self.compute_dtype))
        self._params_replaced()

    def _params_replaced(self) -> None:
        """Called after the whole compute copy was rewritten from outside the optimizer (checkpoint
        load): every rank's buffer is complete."""
