"""Muon / NorMuon optimizer engine.

Parameter routing follows the reference (src/nanoplm/pretraining/optim.py:19-83, 187-205):
1-D tensors and the embedding / un-embedding matrices are updated by AdamW, every other 2-D
hidden matrix by Muon (momentum, optional Nesterov, orthogonalisation of the update by a quintic
Newton-Schulz iteration or the Polar-Express coefficient schedule, decoupled and optionally
"cautious" weight decay); NorMuon additionally normalises each output row of the orthogonalised
update by a running second moment (beta2 0.95) and rescales so the update has unit RMS times a
shape factor.

The reference delegates this to the external `dion` package: Triton Newton-Schulz kernels and, on
several ranks, an all-to-all that hands one whole matrix of every batch of `world` same-shape
matrices to each rank. Here:
* matrices of one shape (one per layer: all QKV projections, all MLP up-projections, ...) are
  stacked and orthogonalised together; every one of the three products of an iteration is ONE
  launch of this package's row-grouped tcgen05 GEMM over the whole stack, so a stack of 16 matrices
  of 1024 x 1024 fills the GPU where a single one would occupy 32 of 148 SMs;
* on several ranks every stack is cut into `world` contiguous runs of matrices: a rank keeps the
  momentum of its run, orthogonalises only that run and the orthogonal factors (bf16) are
  all-gathered; gradients are all-reduced and parameters stay replicated, so what follows the
  gather is elementwise and identical on every rank.

The engine shares storage layout, checkpoint format and API with `ShardedEngine`.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from nanoplm_b200.parallel.engine import AdamWHyper, ShardedEngine

NS_QUINTIC = [(3.4445, -4.7750, 2.0315)] * 5
_PE = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
    (1.891301407787398, -1.2679958271945868, 0.37680408948524835),
    (1.8750014808534479, -1.2500016453999487, 0.3750001645474248),
    (1.875, -1.25, 0.375),
]
POLAR_EXPRESS = [(a / 1.01, b / 1.01 ** 3, c / 1.01 ** 5) for a, b, c in _PE[:-1]] + [_PE[-1]]


def is_embedding_or_unembedding(name: str) -> bool:
    """Token-embedding and output-head tensors stay on AdamW (reference: optim.py:187-205; the
    `embed_tokens` / `shared` names cover T5-style tables)."""
    n = name.lower()
    if n.endswith("decoder.weight") or n.endswith("decoder.bias"):
        return True
    return any(k in n for k in ("embedding", "lm_head", "embed_tokens", "shared"))


_TILE_GROUPS: dict = {}


def _tile_groups(batch: int, rows: int, device) -> torch.Tensor:
    """int32 [batch * rows / 128]: which matrix of the stack every 128-row tile belongs to."""
    key = (batch, rows, str(device))
    t = _TILE_GROUPS.get(key)
    if t is None:
        t = torch.arange(batch, dtype=torch.int32, device=device).repeat_interleave(rows // 128).contiguous()
        _TILE_GROUPS[key] = t
    return t


def _grouped_ok(X: torch.Tensor) -> bool:
    """Stack [B, m, n] whose three Newton-Schulz products fit the row-grouped GEMM kernel."""
    return X.is_cuda and X.dtype == torch.bfloat16 and X.shape[1] % 128 == 0 and X.shape[2] % 64 == 0


def _bmm_nt(a: torch.Tensor, b: torch.Tensor, grouped: bool) -> torch.Tensor:
    """a[i] @ b[i]^T for stacks a [B, m, k], b [B, n, k]."""
    if grouped:
        from nanoplm_b200.ops.moe import gemm_grouped
        B, m, k = a.shape
        return gemm_grouped(a.reshape(B * m, k), b, _tile_groups(B, m, a.device)).view(B, m, b.shape[1])
    return torch.bmm(a, b.transpose(1, 2))


def _bmm_nn(a: torch.Tensor, b: torch.Tensor, grouped: bool) -> torch.Tensor:
    """a[i] @ b[i] for stacks a [B, m, k], b [B, k, n]; b is read as an MN-major operand."""
    if grouped:
        from nanoplm_b200.ops.moe import gemm_grouped
        B, m, k = a.shape
        return gemm_grouped(a.reshape(B * m, k), b, _tile_groups(B, m, a.device), b_mn=True).view(B, m, b.shape[2])
    return torch.bmm(a, b)


def orthogonalize_batched(G: torch.Tensor, coeffs=NS_QUINTIC, eps: float = 1e-7,
                          sumsq: torch.Tensor | None = None) -> torch.Tensor:
    """Approximate polar factor of every matrix of the stack G [B, r, c] by quintic iterations
    X <- aX + (bA + cA^2)X, A = X X^T (bf16 on CUDA, fp32 elsewhere). `sumsq` [B]: squared
    Frobenius norms of the matrices when the caller already has them.

    On the grouped-GEMM path the polynomial is applied through the products only:
    bA + cA^2 = (cA + bI) A and aX + BX = (B + aI) X, so an iteration is three GEMM launches plus
    three small operations on the [B, m, m] Gram stack and never touches X elementwise."""
    dt = torch.bfloat16 if G.is_cuda else torch.float32
    X = G.to(dt)
    transposed = X.shape[1] > X.shape[2]
    if transposed:
        X = X.transpose(1, 2).contiguous()
    nrm = X.float().flatten(1).norm(dim=1) if sumsq is None else sumsq.float().sqrt()
    inv = (1.0 / (nrm * 1.01 + eps)).to(dt)[:, None, None]
    grouped = _grouped_ok(X)
    if grouped:
        X = X.mul_(inv) if (X.data_ptr() != G.data_ptr() or sumsq is not None) else X * inv
        for a, b, c in coeffs:
            A = _bmm_nt(X, X, grouped)                          # X X^T, symmetric [B, m, m]
            Ac = A * c
            Ac.diagonal(dim1=1, dim2=2).add_(b)                 # cA + bI
            Bm = _bmm_nt(Ac, A, grouped)                        # (cA + bI) A^T = bA + cA^2
            Bm.diagonal(dim1=1, dim2=2).add_(a)                 # + aI
            X = _bmm_nn(Bm, X, grouped)                         # aX + (bA + cA^2) X
    else:
        X = X * inv
        for a, b, c in coeffs:
            A = _bmm_nt(X, X, grouped)
            Bm = torch.add(A * b, _bmm_nt(A, A, grouped), alpha=c)
            X = torch.add(_bmm_nn(Bm, X, grouped), X, alpha=a)
    if transposed:
        X = X.transpose(1, 2).contiguous()
    return X


def orthogonalize(G: torch.Tensor, coeffs=NS_QUINTIC, eps: float = 1e-7) -> torch.Tensor:
    """Approximate polar factor of one matrix (see `orthogonalize_batched`)."""
    return orthogonalize_batched(G[None], coeffs, eps)[0]


class _Stack:
    """Muon matrices of one shape; `lo:hi` is the run this rank orthogonalises."""

    def __init__(self, slots, rank: int, world: int):
        self.slots = slots
        self.shape = tuple(slots[0].shape)
        n = len(slots)
        self.even = world > 1 and n % world == 0
        if world == 1:
            self.lo, self.hi = 0, n
        elif self.even:
            self.lo, self.hi = rank * (n // world), (rank + 1) * (n // world)
        else:                                   # uneven: near-equal contiguous runs, exchanged by all-reduce
            self.lo, self.hi = rank * n // world, (rank + 1) * n // world

    def offsets(self, device, own: bool) -> torch.Tensor:
        """int64 flat offsets of this rank's run (own) or of all matrices of the stack."""
        key = "_off_own" if own else "_off_all"
        t = getattr(self, key, None)
        if t is None:
            sl = self.slots[self.lo:self.hi] if own else self.slots
            t = torch.tensor([s.offset for s in sl], dtype=torch.int64, device=device)
            setattr(self, key, t)
        return t

    def views(self, flat: torch.Tensor, lo: int = 0, hi: int | None = None):
        return [flat[s.offset:s.offset + s.numel].view(s.shape) for s in self.slots[lo:hi]]


class MuonEngine(ShardedEngine):
    def __init__(self, model, hyper: AdamWHyper, cfg, device, process_group=None, fused_comm: bool | None = None):
        compute = torch.bfloat16 if (getattr(cfg, "bf16", True) and torch.device(device).type == "cuda") else torch.float32
        if fused_comm is None:
            fused_comm = bool(getattr(cfg, "fused_comm", True))
        super().__init__(model, hyper, device, process_group, compute_dtype=compute, fused_comm=fused_comm)
        # replicated parameters and AdamW state: full-size buffers on every rank; the Muon momentum
        # lives in the same flat buffer but only the entries of matrices this rank owns are used
        dev = self.device
        self.master = self._gather_full(self.master).clone()
        self.exp_avg = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.shard, self.lo, self.hi = self.total, 0, self.total
        self.normuon = str(cfg.optimizer).lower() == "normuon"
        self.mu = float(cfg.muon_momentum)
        self.nesterov = bool(cfg.muon_nesterov)
        self.muon_lr0, self.adam_lr0 = float(cfg.muon_learning_rate), float(cfg.adam_learning_rate)
        self.muon_wd = float(cfg.muon_weight_decay)
        self.cautious = bool(cfg.muon_cautious_weight_decay)
        self.muon_eps = float(cfg.muon_eps)
        self.coeffs = POLAR_EXPRESS if cfg.muon_use_polar_express else NS_QUINTIC
        self.muon_slots = [s for s in self.slots if len(s.shape) == 2 and not is_embedding_or_unembedding(s.name)]
        if not self.muon_slots:
            raise ValueError("No eligible matrix parameters found for Muon (expected 2D hidden-layer weights).")
        muon_ids = {id(s) for s in self.muon_slots}
        self.adam_slots = [s for s in self.slots if id(s) not in muon_ids]
        by_shape: dict = {}
        for s in self.muon_slots:
            by_shape.setdefault(tuple(s.shape), []).append(s)
        self.stacks = [_Stack(v, self.rank, self.world) for v in by_shape.values()]
        self.row_second_moment = {s.name: torch.zeros(s.shape[0], dtype=torch.float32, device=dev)
                                  for s in self.muon_slots} if self.normuon else {}
        self.muon_lr = self.muon_lr0
        # CUDA kernels for the elementwise parts: matrices are whole float4 runs at aligned offsets
        self._kernels = self.kernel_opt and all(s.numel % 4 == 0 and s.offset % 4 == 0 for s in self.muon_slots)
        self._gsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._gscale = 1.0
        self._adam_table = None
        # peer-memory path: gradients pulled by the matrix owners, updates pushed to every rank
        if self.fused is not None:
            usable = self._kernels and all(s.numel % 8 == 0 for s in self.muon_slots)
            ok = torch.tensor([1.0 if usable else 0.0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.pg)
            if ok.item() < 1:
                self.fused = None
            else:
                self.fused.setup(self.stacks, self.adam_slots)

    def _make_fused(self, sym):
        from nanoplm_b200.comm.fused_optimizer import MuonPeerStep
        return MuonPeerStep(self, *sym)

    def begin_last_microstep(self) -> None:
        """The Muon step reduces whole matrices after the backward pass: nothing to arm."""

    # ---- checkpoint helpers ------------------------------------------------------------------
    def _owned(self):
        return [s for st in self.stacks for s in st.slots[st.lo:st.hi]]

    def _gather_full(self, t):
        if t.numel() != self.total:
            return super()._gather_full(t)
        if t is not getattr(self, "exp_avg", None) or not self.distributed:
            return t                                  # replicated: already complete on every rank
        # Muon momentum: every matrix from the rank that owns it, AdamW entries from this rank
        full = torch.zeros_like(t)
        for s in self._owned():
            full[s.offset:s.offset + s.numel] = t[s.offset:s.offset + s.numel]
        dist.all_reduce(full, group=self.pg)
        for s in self.adam_slots:
            full[s.offset:s.offset + s.numel] = t[s.offset:s.offset + s.numel]
        return full

    def _drop_unowned_momentum(self) -> None:
        owned = {id(s) for s in self._owned()}
        for s in self.muon_slots:
            if id(s) not in owned:
                self.exp_avg[s.offset:s.offset + s.numel].zero_()

    def optimizer_state_dict(self) -> dict:
        sd = super().optimizer_state_dict()
        if self.normuon:
            rows = {}
            owned = {id(s) for s in self._owned()}
            for s in self.muon_slots:
                v = self.row_second_moment[s.name]
                v = v.clone() if id(s) in owned else torch.zeros_like(v)
                if self.distributed:
                    dist.all_reduce(v, group=self.pg)
                rows[s.name] = v.cpu()
            sd["normuon_row_second_moment"] = rows
        return sd

    def load_optimizer_state_dict(self, sd: dict) -> None:
        super().load_optimizer_state_dict(sd)
        self._drop_unowned_momentum()
        for name, v in (sd.get("normuon_row_second_moment") or {}).items():
            if name in self.row_second_moment:
                self.row_second_moment[name].copy_(v)

    # ---- the step ----------------------------------------------------------------------------
    def _adamw_group(self, slots, g_all, lr: float, wd: float, bc1: float, bc2: float) -> None:
        if not slots:
            return
        h = self.hyper
        view = lambda flat: [flat[s.offset:s.offset + s.numel] for s in slots]
        p, m, v, g = view(self.master), view(self.exp_avg), view(self.exp_avg_sq), view(g_all)
        if wd:
            torch._foreach_mul_(p, 1 - lr * wd)
        torch._foreach_mul_(m, h.beta1)
        torch._foreach_add_(m, g, alpha=1 - h.beta1)
        torch._foreach_mul_(v, h.beta2)
        torch._foreach_addcmul_(v, g, g, value=1 - h.beta2)
        den = torch._foreach_sqrt(v)
        torch._foreach_div_(den, math.sqrt(bc2))
        torch._foreach_add_(den, h.eps)
        torch._foreach_addcdiv_(p, m, den, value=-lr / bc1)

    def _orthogonal_updates(self, st: _Stack, g_all: torch.Tensor) -> torch.Tensor:
        """Orthogonalised (and, for NorMuon, row-normalised) updates of the whole stack
        [n, r, c]; this rank computes its run, the others arrive by all-gather."""
        n = len(st.slots)
        dt = torch.bfloat16 if self.on_cuda else torch.float32
        peer = self.fused is not None
        if peer:
            index = self.stacks.index(st)
            O = self.fused.stack_buffers[index].tensor.view((n,) + st.shape)
        elif not st.even and self.distributed:
            O = torch.zeros((n,) + st.shape, dtype=dt, device=self.device)
        else:
            O = torch.empty((n,) + st.shape, dtype=dt, device=self.device)
        if st.hi > st.lo:
            if self._kernels:
                from nanoplm_b200.ops import kernels as K
                k, numel = st.hi - st.lo, st.slots[0].numel
                upd = torch.empty((k,) + st.shape, dtype=torch.bfloat16, device=self.device)
                usq = torch.zeros(k, dtype=torch.float32, device=self.device)
                K.muon_momentum_(g_all, self.exp_avg, st.offsets(self.device, True), numel, upd, usq, self._gsq,
                                 self._gscale, self.hyper.max_grad_norm, self.mu, self.nesterov)
                mine = orthogonalize_batched(upd, self.coeffs, self.muon_eps, sumsq=usq)
            else:
                g = st.views(g_all, st.lo, st.hi)
                m = st.views(self.exp_avg, st.lo, st.hi)
                torch._foreach_mul_(m, self.mu)
                torch._foreach_add_(m, g)
                upd = torch.stack(torch._foreach_add(g, m, alpha=self.mu) if self.nesterov else m)
                mine = orthogonalize_batched(upd, self.coeffs, self.muon_eps)
            if self.normuon:
                mine = mine.float()
                v = torch.stack([self.row_second_moment[s.name] for s in st.slots[st.lo:st.hi]])
                v.mul_(0.95).add_(mine.pow(2).mean(dim=2), alpha=0.05)
                for s, row in zip(st.slots[st.lo:st.hi], v):
                    self.row_second_moment[s.name].copy_(row)
                mine = mine / (v.sqrt()[:, :, None] + self.muon_eps)
                scale = 0.2 * math.sqrt(mine[0].numel()) / (mine.flatten(1).norm(dim=1) + self.muon_eps)
                mine = mine * scale[:, None, None]                                        # rms_norm scaling
            O[st.lo:st.hi] = mine.to(dt)
        if peer:
            self.fused.push_run(index, st.lo, st.hi - st.lo, st.slots[0].numel)   # visible after the next barrier
        elif self.distributed:
            if st.even and self.on_cuda:
                dist.all_gather_into_tensor(O, O[st.lo:st.hi].clone(), group=self.pg)
            elif st.even:
                parts = [torch.empty_like(O[st.lo:st.hi]) for _ in range(self.world)]
                dist.all_gather(parts, O[st.lo:st.hi].contiguous(), group=self.pg)
                O = torch.cat(parts)
            else:
                dist.all_reduce(O, group=self.pg)
        return O

    @torch.no_grad()
    def step(self, lr: float, grad_accum: int = 1) -> torch.Tensor:
        self.collect_autograd_grads()
        self.step_count += 1
        from nanoplm_b200.parallel.engine import _invalidate_fp8_weights
        _invalidate_fp8_weights()
        if self.distributed and self.fused is None:
            dist.all_reduce(self.main_grad, group=self.pg)
        scale = 1.0 / (grad_accum * self.world)
        h, t = self.hyper, self.step_count
        self.muon_lr = self.muon_lr0 * (lr / self.adam_lr0 if self.adam_lr0 > 0 else 1.0)   # same schedule shape
        bc1, bc2 = 1 - h.beta1 ** t, 1 - h.beta2 ** t
        if self._kernels:
            return self._step_kernels(lr, scale, bc1, bc2)
        g_all = self.main_grad.mul_(scale)
        norm = g_all.norm()
        if self.hyper.max_grad_norm > 0:
            g_all.mul_(torch.clamp(self.hyper.max_grad_norm / (norm + 1e-6), max=1.0))
        for st in self.stacks:
            O = self._orthogonal_updates(st, g_all).float()
            p_views = st.views(self.master)
            p = torch.stack(p_views)
            if self.muon_wd > 0:
                if self.cautious:
                    p.sub_(self.muon_lr * self.muon_wd * p * ((O * p) > 0))
                else:
                    p.mul_(1 - self.muon_lr * self.muon_wd)
            p.sub_(self.muon_lr * O)
            torch._foreach_copy_(p_views, list(p.unbind(0)))
        self._adamw_group([s for s in self.adam_slots if s.decay], g_all, lr, h.weight_decay, bc1, bc2)
        self._adamw_group([s for s in self.adam_slots if not s.decay], g_all, lr, 0.0, bc1, bc2)
        self.flat_params.copy_(self.master)
        self.main_grad.zero_()
        return norm

    def _step_kernels(self, lr: float, scale: float, bc1: float, bc2: float) -> torch.Tensor:
        """CUDA path: gradient scaling and clipping are folded into the kernels that read the
        gradient (global norm read on the device), one kernel each for the momentum and the
        parameter update of a stack, one for all AdamW tensors."""
        from nanoplm_b200.ops import kernels as K
        h = self.hyper
        if self.fused is not None:
            grad = self.fused.reduce(self._owned(), self._gsq)
        else:
            grad = self.main_grad
            self._gsq.zero_()
            K.sumsq_(grad, self._gsq)
        self._gscale = scale
        norm = self._gsq.sqrt() * scale
        p16 = self.flat_params if self.flat_params.dtype == torch.bfloat16 else None
        updates = [self._orthogonal_updates(st, grad) for st in self.stacks]
        if self.fused is not None:
            self.fused.barrier()     # every owner's updates have landed; peers are done reading my gradients
        for st, O in zip(self.stacks, updates):
            K.muon_apply_(self.master, p16, st.offsets(self.device, False), st.slots[0].numel, O.contiguous(),
                          self.muon_lr, self.muon_wd, self.cautious)
        if self.adam_slots:
            if self._adam_table is None:
                dev = self.device
                self._adam_table = (
                    torch.tensor([s.offset for s in self.adam_slots], dtype=torch.int64, device=dev),
                    torch.tensor([s.numel for s in self.adam_slots], dtype=torch.int64, device=dev),
                    torch.tensor([int(s.decay) for s in self.adam_slots], dtype=torch.int32, device=dev),
                    max(s.numel for s in self.adam_slots))
            off, num, dec, mx = self._adam_table
            K.adamw_slots_(self.master, self.exp_avg, self.exp_avg_sq, grad, p16, off, num, dec, mx,
                           self._gsq, scale, h.max_grad_norm, lr, h.beta1, h.beta2, h.eps, h.weight_decay, bc1, bc2)
        if p16 is None:
            self.flat_params.copy_(self.master)
        self.main_grad.zero_()
        return norm


def is_muon_optimizer(engine) -> bool:
    """True for the Muon / NorMuon engine (used to decide which learning rates to log;
    reference: pretraining/optim.py:10-17)."""
    return isinstance(engine, MuonEngine)
