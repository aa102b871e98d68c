"""Data parallelism with SHARDED PARAMETERS: what the reference gets from FSDP2's `fully_shard`
per layer (src/nanoplm/pretraining/pure_pipeline.py:479-506: parameters, gradients and optimizer
state split over the ranks, all-gather before use, reduce-scatter after the backward pass).

`ShardedEngine` shards the optimizer state only and pushes every updated parameter to every rank at
the end of the step. Here the persistent state of a weight matrix is split by ROWS: rank r owns rows
[r n/N, (r+1) n/N) of every large matrix: its fp32 master copy, its Adam moments and its bf16 values.
After an optimizer step a rank's compute buffer holds only its own rows up to date; the other rows
arrive INSIDE the first GEMM that multiplies by the matrix in the next forward pass
(`nplm_gemm_bf16_ag`: the epilogue warps pull the peers' row blocks over NVLink while the tensor
cores start on the local block; QKV with the RoPE epilogue, MLP-up with the SwiGLU epilogue, the two
output projections with the residual epilogue). The gathered matrix stays in the buffer and serves
the remaining micro-steps and the backward GEMMs until the next optimizer step (the reference runs
FSDP2 with reshard_after_forward=False in the same way, pure_pipeline.py:691-692).

Gradients: every rank keeps the full fp32 gradient buffer the weight-gradient GEMMs add into; rank r
reduces ITS row block of a matrix from all peers (plain P2P loads) as soon as the matrix's gradient
kernel of the last micro-step has been launched, so every rank reduces 1/N of every matrix while
the backward pass of the earlier layers is still running. AdamW then updates the owned rows in
place; nothing is pushed.

Tensors that no GEMM gathers (embedding, norms, biases, matrices whose row count does not split into
whole 128-row tiles) have one owner each (dealt round-robin); the owner updates them and pushes the
few bytes to every rank.

Without the peer-memory path (CPU ranks over gloo, or `fused_comm` off) the same ownership is used
with library collectives: all-reduce of the gradients, AdamW on the owned pieces, one all-reduce of
a buffer holding every rank's updated pieces.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .engine import ParamSlot, ShardedEngine, _invalidate_fp8_weights, _round_up

TILE_ROWS = 128      # a row block must hold whole GEMM tiles


@dataclass
class Piece:
    """A contiguous range [a, b) of the flat index space with one owner."""
    slot: ParamSlot
    a: int
    b: int
    owner: int
    local: int        # offset inside the owner's optimizer-state arrays
    gathered: bool    # True: a row block the consuming GEMM gathers; False: pushed to every rank


class GatherState:
    """Attached to a parameter as `._ag`: tells `ops.kernels.gemm` that the next forward GEMM with
    this weight has to gather the other ranks' row blocks (see `gemm_ag`)."""

    def __init__(self, ptrs, rank: int, world: int, flags: torch.Tensor):
        self.ptrs, self.rank, self.world, self.flags = ptrs, rank, world, flags
        self.stale = False
        self.peer_views = None      # set by the engine: callable r -> that rank's buffer of this tensor

    def gather_now(self, w: torch.Tensor) -> None:
        """Explicit gather for consumers other than a qualifying forward GEMM (copies over NVLink)."""
        if not self.stale:
            return
        rows = w.shape[0] // self.world
        for r in range(self.world):
            if r != self.rank:
                w[r * rows:(r + 1) * rows].copy_(self.peer_views(r)[r * rows:(r + 1) * rows])
        self.stale = False


class ParamShardedEngine(ShardedEngine):
    def __init__(self, model, hyper, device, process_group=None, compute_dtype=torch.bfloat16,
                 fused_comm: bool = True, exclude=()):
        super().__init__(model, hyper, device, process_group, compute_dtype, fused_comm, exclude)
        self._attach_gather_states()

    # ---- ownership ------------------------------------------------------------------------------
    def _plan_ownership(self) -> None:
        w = self.world
        self.pieces: list[Piece] = []
        fill = [0] * w
        small = 0
        for s in self.slots:
            rows = s.shape[0] if len(s.shape) == 2 else 0
            splits = (w > 1 and rows > 0 and s.name not in self._shared_names and rows % w == 0
                      and (rows // w) % TILE_ROWS == 0)
            if splits:
                blk = s.numel // w
                for r in range(w):
                    self.pieces.append(Piece(s, s.offset + r * blk, s.offset + (r + 1) * blk, r, fill[r], True))
                    fill[r] = _round_up(fill[r] + blk, 8)
            else:
                r = small % w
                small += 1
                n = _round_up(s.numel, 8)        # slots start on 64-element boundaries: the pad is ours
                self.pieces.append(Piece(s, s.offset, s.offset + n, r, fill[r], False))
                fill[r] = _round_up(fill[r] + n, 8)
        self.shard = _round_up(max(max(fill), 64), 64)
        self.lo, self.hi = 0, 0                # no contiguous slice in this layout
        self.mine = [p for p in self.pieces if p.owner == self.rank]

    def _take_local(self, full: torch.Tensor) -> torch.Tensor:
        local = torch.zeros(self.shard, dtype=full.dtype, device=full.device)
        for p in self.mine:
            local[p.local:p.local + (p.b - p.a)] = full[p.a:p.b]
        return local

    def _gather_full(self, local: torch.Tensor) -> torch.Tensor:
        if not self.distributed:
            parts = [local]
        elif self.on_cuda:
            flat = torch.empty(self.world * self.shard, dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(flat, local.contiguous(), group=self.pg)
            parts = list(flat.view(self.world, self.shard))
        else:
            parts = [torch.empty_like(local) for _ in range(self.world)]
            dist.all_gather(parts, local.contiguous(), group=self.pg)
        full = torch.zeros(self.total, dtype=local.dtype, device=local.device)
        for p in self.pieces:
            full[p.a:p.b] = parts[p.owner][p.local:p.local + (p.b - p.a)]
        return full

    def _make_fused(self, sym):
        from nanoplm_b200.comm.fused_optimizer import ParamShardedStep
        return ParamShardedStep(self, *sym)

    def _attach_gather_states(self) -> None:
        self.gather_states: list[GatherState] = []
        if self.fused is None:
            return
        flags = torch.zeros(8, dtype=torch.int32, device=self.device)
        base = self.fused.params           # SymmetricBuffer of the compute copy
        from nanoplm_b200.comm.fused_optimizer import _ptr_array
        seen = set()
        for p in self.pieces:
            if not p.gathered or id(p.slot) in seen:
                continue
            seen.add(id(p.slot))
            s = p.slot
            st = GatherState(_ptr_array([ptr + 2 * s.offset for ptr in base.ptrs]), self.rank, self.world, flags)
            handle, off, shape = base.handle, s.offset, s.shape
            st.peer_views = (lambda r, handle=handle, off=off, shape=shape:
                             handle.get_buffer(r, (off + shape[0] * shape[1],), torch.bfloat16)[off:].view(shape))
            s.param._ag = st
            self.gather_states.append(st)

    def _params_replaced(self) -> None:
        for st in getattr(self, "gather_states", []):
            st.stale = False

    def gathered_parameter_bytes(self) -> int:
        """bf16 bytes a rank receives per optimizer step through the gathering GEMMs."""
        n = sum(p.b - p.a for p in self.pieces if p.gathered and p.owner != self.rank)
        return 2 * n

    # ---- optimizer step -------------------------------------------------------------------------
    def step(self, lr: float, grad_accum: int = 1, extra_sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
        if extra_sumsq is not None:
            raise ValueError("extra_sumsq is not supported with sharded parameters")
        self.collect_autograd_grads()
        self.step_count += 1
        _invalidate_fp8_weights()
        grad_scale = 1.0 / (grad_accum * self.world)
        self._fill_hyper(lr, grad_scale)
        if self.fused is not None:
            from nanoplm_b200.ops import functional as ops
            ops.set_wgrad_ready_callback(None)
            norm = self.fused.step(lr, grad_scale)
            for st in self.gather_states:      # the peers' rows of every gathered matrix are out of date
                st.stale = True
            return norm
        # ---- library collectives, same ownership ------------------------------------------------
        if self.distributed:
            dist.all_reduce(self.main_grad, op=dist.ReduceOp.SUM, group=self.pg)
        grad = self._take_local(self.main_grad)
        self._sumsq.zero_()
        self._sumsq += grad.double().pow(2).sum().float()
        if self.distributed:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=self.pg)
        grad_norm = self._sumsq.sqrt() * grad_scale
        new_local = torch.zeros(self.shard, dtype=self.flat_params.dtype, device=self.device)
        for p in self.mine:
            sl = slice(p.local, p.local + (p.b - p.a))
            group = 0 if p.slot.decay else 1
            if self.kernel_opt:
                from nanoplm_b200.ops import kernels as K
                K.adamw_(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], grad[sl], new_local[sl],
                         self._hyper_dev[group], self._sumsq, zero_grad=False)
            else:
                self._adamw_cpu(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], grad[sl], new_local[sl],
                                group, lr, grad_scale)
        self.flat_params.copy_(self._gather_full(new_local))
        self.main_grad.zero_()
        return grad_norm

    # ---- sharded checkpoint fast path: the layout differs from the slice layout --------------------
    def shard_state(self) -> dict:
        st = super().shard_state()
        st["layout"] = "row-blocks"
        return st

    def load_shard_state(self, st: dict) -> None:
        if st.get("layout") != "row-blocks":
            raise ValueError("sharded checkpoint was written by an engine with a different ownership layout")
        super().load_shard_state(st)
