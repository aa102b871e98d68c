"""Muon / NorMuon optimizer engine.

Parameter routing follows the reference (src/nanoplm/pretraining/optim.py:19-83, 187-205):
1-D tensors and the embedding / un-embedding matrices are updated by AdamW, every other 2-D
hidden matrix by Muon (momentum, optional Nesterov, orthogonalisation of the update by a quintic
Newton-Schulz iteration or the Polar-Express coefficient schedule, decoupled and optionally
"cautious" weight decay); NorMuon additionally normalises each output row of the orthogonalised
update by a running second moment (beta2 0.95) and rescales so the update has unit RMS times a
shape factor. The reference delegates this to the external `dion` package (Triton Newton-Schulz,
sharded all-to-all); here the iterations are plain matrix products on this package's GEMM kernel,
gradients are all-reduced and every rank applies the same (replicated) update: at 169 M parameters
the full orthogonalisation costs a few milliseconds per optimizer step.

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
    n = name.lower()
    return any(k in n for k in ("tok_embeddings", "embed_tokens", "word_embeddings", "decoder", "lm_head", "shared"))


def _mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b^T for bf16 2-D operands: tcgen05 GEMM on CUDA (both K-major), torch elsewhere."""
    if a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.shape[0] % 8 == 0 and b.shape[0] % 8 == 0:
        from nanoplm_b200.ops import kernels as K
        return K.gemm(a.contiguous(), b.contiguous())
    return a @ b.t()


def _mm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b for bf16 2-D operands; on CUDA b is consumed as an MN-major operand, no transpose."""
    if (a.is_cuda and a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.shape[0] % 8 == 0
            and b.shape[1] % 64 == 0 and b.is_contiguous()):
        from nanoplm_b200.ops import kernels as K
        return K.gemm(a.contiguous(), b, b_mn=True)
    return a @ b


def orthogonalize(G: torch.Tensor, coeffs=NS_QUINTIC, eps: float = 1e-7) -> torch.Tensor:
    """Approximate polar factor of G by quintic iterations X <- aX + (bA + cA^2)X, A = X X^T."""
    dt = torch.bfloat16 if G.is_cuda else torch.float32
    X = G.to(dt)
    transposed = X.shape[0] > X.shape[1]
    if transposed:
        X = X.t().contiguous()
    X = X / (X.float().norm() * 1.01 + eps).to(dt)
    for a, b, c in coeffs:
        A = _mm(X, X)                                   # X X^T          [m, m], symmetric
        B = b * A + c * _mm(A, A)                       # A A^T = A^2
        X = a * X + _mm_nn(B, X)                        # B X
    if transposed:
        X = X.t().contiguous()
    return X


class MuonEngine(ShardedEngine):
    def __init__(self, model, hyper: AdamWHyper, cfg, device, process_group=None):
        compute = torch.bfloat16 if (getattr(cfg, "bf16", True) and torch.device(device).type == "cuda") else torch.float32
        super().__init__(model, hyper, device, process_group, compute_dtype=compute, fused_comm=False)
        # replicated optimizer state: full-size buffers on every rank
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
        self._muon_ids = {id(s) for s in self.slots if s in self.muon_slots}
        self.row_second_moment = {s.name: torch.zeros(s.shape[0], dtype=torch.float32, device=dev)
                                  for s in self.muon_slots} if self.normuon else {}
        self.muon_lr = self.muon_lr0

    def _gather_full(self, t):                       # state is already complete on every rank
        if t.numel() == self.total:
            return t
        return super()._gather_full(t)

    @torch.no_grad()
    def step(self, lr: float, grad_accum: int = 1) -> torch.Tensor:
        self.collect_autograd_grads()
        self.step_count += 1
        from nanoplm_b200.parallel.engine import _invalidate_fp8_weights
        _invalidate_fp8_weights()
        if self.distributed:
            dist.all_reduce(self.main_grad, group=self.pg)
        scale = 1.0 / (grad_accum * self.world)
        g_all = self.main_grad.mul_(scale)
        norm = g_all.norm()
        if self.hyper.max_grad_norm > 0:
            g_all.mul_(torch.clamp(self.hyper.max_grad_norm / (norm + 1e-6), max=1.0))
        h, t = self.hyper, self.step_count
        self.muon_lr = self.muon_lr0 * (lr / self.adam_lr0 if self.adam_lr0 > 0 else 1.0)   # same schedule shape
        bc1, bc2 = 1 - h.beta1 ** t, 1 - h.beta2 ** t
        for s in self.slots:
            sl = slice(s.offset, s.offset + s.numel)
            g, p = g_all[sl], self.master[sl]
            if id(s) in self._muon_ids:
                m = self.exp_avg[sl]
                m.mul_(self.mu).add_(g)
                upd = (g + self.mu * m) if self.nesterov else m
                O = orthogonalize(upd.view(s.shape), self.coeffs, self.muon_eps).float()
                if self.normuon:
                    v = self.row_second_moment[s.name]
                    v.mul_(0.95).add_(O.pow(2).mean(dim=1), alpha=0.05)
                    O = O / (v.sqrt()[:, None] + self.muon_eps)
                    O = O * (0.2 * math.sqrt(O.numel()) / (O.norm() + self.muon_eps))      # rms_norm scaling
                O = O.reshape(-1)
                if self.muon_wd > 0:
                    if self.cautious:
                        p.sub_(self.muon_lr * self.muon_wd * p * ((O * p) > 0))
                    else:
                        p.mul_(1 - self.muon_lr * self.muon_wd)
                p.sub_(self.muon_lr * O)
            else:
                m, v = self.exp_avg[sl], self.exp_avg_sq[sl]
                wd = h.weight_decay if s.decay else 0.0
                p.mul_(1 - lr * wd)
                m.mul_(h.beta1).add_(g, alpha=1 - h.beta1)
                v.mul_(h.beta2).addcmul_(g, g, value=1 - h.beta2)
                p.addcdiv_(m, (v.sqrt() / math.sqrt(bc2)).add_(h.eps), value=-lr / bc1)
            self.flat_params[sl] = p.to(self.flat_params.dtype)
        self.main_grad.zero_()
        return norm


def is_muon_optimizer(engine) -> bool:
    """True for the Muon / NorMuon engine (used to decide which learning rates to log;
    reference: pretraining/optim.py:10-17)."""
    return isinstance(engine, MuonEngine)
