"""Device-side mixture-of-experts pipeline: router top-k, planning, token dispatch, grouped expert
GEMMs and combine, with autograd. Kernels: nanoplm_b200/csrc/moe.cu and the grouped forms of
nanoplm_b200/csrc/gemm_tcgen05.cu. The reference has no MoE layers.

Nothing here synchronises with the host: expert counts stay on the device, every buffer is sized
for the worst case (or a capacity factor with expert parallelism) and unused 128-row tiles are
skipped inside the grouped GEMM.

Expert parallelism (`MoEComm` with world > 1) keeps the expert-major buffers in symmetric memory:
token rows are pushed straight into the owner rank's buffer and pulled back from it with plain
peer loads / stores; flag barriers (bounded waits) order the phases.
"""
from __future__ import annotations

from ctypes import c_double, c_int, c_longlong, c_uint, c_void_p

import torch

from . import kernels as K
from ._lib import check_rc, count_launch, lib, ptr, status_word, stream_ptr

_BF16 = torch.bfloat16


def _ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = c_void_p(int(p))
    return arr


# ------------------------------------------------------------------------------ raw kernels
def router_topk(logits: torch.Tensor, k: int):
    """logits bf16 [T,E] -> probs fp32 [T,E], gates fp32 [T,k], experts int32 [T,k], probsum fp32 [E],
    counts int32 [E]."""
    T, E = logits.shape
    dev = logits.device
    probs = torch.empty((T, E), dtype=torch.float32, device=dev)
    gates = torch.empty((T, k), dtype=torch.float32, device=dev)
    experts = torch.empty((T, k), dtype=torch.int32, device=dev)
    probsum = torch.zeros(E, dtype=torch.float32, device=dev)
    counts = torch.zeros(E, dtype=torch.int32, device=dev)
    rc = lib("moe").nplm_router_topk(ptr(logits), c_int(T), c_int(E), c_int(k), ptr(probs), ptr(gates),
                                     ptr(experts), ptr(probsum), ptr(counts), stream_ptr())
    check_rc(rc, "router_topk")
    count_launch()
    return probs, gates, experts, probsum, counts


def router_bwd(probs, gates, experts, d_gates, aux_grad):
    T, E = probs.shape
    k = gates.shape[1]
    dlogits = torch.empty((T, E), dtype=_BF16, device=probs.device)
    rc = lib("moe").nplm_router_bwd(ptr(probs), ptr(gates), ptr(experts), ptr(d_gates), ptr(aux_grad),
                                    c_int(T), c_int(E), c_int(k), ptr(dlogits), stream_ptr())
    check_rc(rc, "router_bwd")
    count_launch()
    return dlogits


def gemm_grouped(a, b, tile_group, *, b_mn=False, epi=K.EPI_STORE, aux=None, bn=None, out=None,
                 arrive=None, expect=None):
    """Row-grouped GEMM. a [P,K] bf16 (P multiple of 128), b [G, N, K] (b_mn False) or [G, K, N]
    (b_mn True), tile_group int32 [P/128]. Returns [P, N] (N/2 wide for EPI_SWIGLU).
    arrive / expect (int32 [P/128] each, both or neither): the rows of `a` are being stored by other GPUs;
    a tile is loaded once its arrival counter has reached its expected row count."""
    P, Kd = a.shape
    G = b.shape[0]
    if b_mn:
        N, rows_per_group = b.shape[2], b.shape[1]
        if b.shape[1] != Kd:
            raise ValueError("inner dims differ")
    else:
        N, rows_per_group = b.shape[1], b.shape[1]
        if b.shape[2] != Kd:
            raise ValueError("inner dims differ")
    if P % 128 or tile_group.numel() < P // 128:
        raise ValueError("grouped GEMM rows must be whole 128-row tiles described by tile_group")
    out_cols = N // 2 if epi == K.EPI_SWIGLU else N
    if out is None:
        out = torch.empty((P, out_cols), dtype=_BF16, device=a.device)
    elif tuple(out.shape) != (P, out_cols) or out.dtype != _BF16:
        raise ValueError("out has the wrong shape or dtype")
    b2 = b.reshape(-1, b.shape[2])
    if bn is None:
        bn = 256 if (N >= 256 or epi == K.EPI_SWIGLU) else 128
    ldr = aux.stride(0) if aux is not None else 0
    if (arrive is None) != (expect is None):
        raise ValueError("arrive and expect go together")
    if arrive is not None and (arrive.numel() < P // 128 or expect.numel() < P // 128
                               or arrive.dtype != torch.int32 or expect.dtype != torch.int32):
        raise ValueError("arrive / expect must be int32 with one entry per 128-row tile")
    rc = lib("gemm_tcgen05").nplm_gemm_bf16_grouped_gated(
        ptr(a), ptr(b2), ptr(out), ptr(aux), c_int(P), c_int(N), c_int(Kd), c_int(a.stride(0)),
        c_int(b2.stride(0)), c_int(out.stride(0)), c_int(ldr), c_int(int(b_mn)), c_int(epi), c_int(bn),
        c_int(G), ptr(tile_group), c_int(rows_per_group), ptr(arrive), ptr(expect),
        ptr(status_word(a.device)), stream_ptr())
    check_rc(rc, "gemm_bf16_grouped")
    count_launch()
    return out


def gemm_grouped_wgrad(dy, x, group_off, out, accumulate=True):
    """out[g] (fp32 [G, N, Kin]) (+)= dy[rows_g]^T x[rows_g]; rows_g from group_off int32 [G+1]."""
    P, N = dy.shape
    Kin = x.shape[1]
    G = out.shape[0]
    rc = lib("gemm_tcgen05").nplm_gemm_bf16_grouped_wgrad(
        ptr(dy), ptr(x), ptr(out), c_int(N), c_int(Kin), c_int(P), c_int(dy.stride(0)), c_int(x.stride(0)),
        c_int(Kin), c_int(int(accumulate)), c_int(256 if Kin >= 256 else 128), c_int(G), ptr(group_off),
        c_longlong(N * Kin), ptr(status_word(dy.device)), stream_ptr())
    check_rc(rc, "gemm_bf16_grouped_wgrad")
    count_launch()
    return out


# ------------------------------------------------------------------------------ communicator
class MoEComm:
    """Buffers and peer pointers of one MoE layer.

    world == 1: buffers are ordinary tensors allocated per call. world > 1: three expert-major
    buffers of `capacity_rows` rows, the count table and the barrier flags live in symmetric memory
    (allocated once, identical on every rank of `group`)."""

    def __init__(self, hidden: int, num_experts: int, top_k: int, group=None, capacity_factor: float = 0.0,
                 barrier_timeout_s: float = 20.0):
        self.C, self.E, self.k = hidden, num_experts, top_k
        self.group = group
        self.world, self.rank = 1, 0
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.E % self.world:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.El = self.E // self.world
        # rows a rank's buffers hold, in units of its even share of the assignments. `world` is the
        # worst case (every row of every rank lands here: nothing can be dropped); 0 picks that up to
        # four shares, which bounds the buffers at 8 and more ranks, where rows past them are
        # dropped and counted
        self.capacity_factor = float(capacity_factor) if capacity_factor and capacity_factor > 0 else float(
            min(max(self.world, 1), 4))
        self.timeout = barrier_timeout_s
        self.epoch = 0
        self._sym = None
        self._cap = 0
        self._dropped = None      # int32 device counter: expert rows dropped for lack of buffer room
        # expert parallelism: the up-projection starts tile by tile on arrival counters instead of after a
        # barrier over all ranks (NPLM_MOE_GATED=0 restores the barrier)
        import os
        self.gated_dispatch = os.environ.get("NPLM_MOE_GATED", "1") != "0"
        # the same for the gradient rows of the backward pass (NPLM_MOE_GATED_BWD=0: flag barriers there)
        self.gated_backward = self.gated_dispatch and os.environ.get("NPLM_MOE_GATED_BWD", "1") != "0"

    def dropped_counter(self, device) -> torch.Tensor:
        if self._dropped is None:
            self._dropped = torch.zeros(1, dtype=torch.int32, device=device)
        return self._dropped

    def dropped_rows(self) -> int:
        """Assignments dropped so far because a rank's experts received more rows than its buffer
        holds (synchronises)."""
        return 0 if self._dropped is None else int(self._dropped.item())

    def capacity(self, n_assign: int) -> int:
        if self.world == 1:
            rows = n_assign + self.El * 127
        else:
            rows = int(self.capacity_factor * n_assign) + self.El * 127
        return (rows + 127) // 128 * 128

    def _ensure_symmetric(self, cap: int, device):
        """Allocates the symmetric buffers on first use. Symmetric allocations must have the same
        size on every rank, so the capacity is the maximum over the ranks of the first request (one
        host-synchronising all-reduce, once) plus a quarter: micro-batches whose padding tail has been
        cut off differ in length. A later, larger request keeps the buffers: the capacity is a bound
        on the rows that may LAND on a rank (capacity_factor times the even share), rows past it are
        dropped and counted by the plan kernel."""
        if self._sym is not None:
            return
        cap = (cap + cap // 4 + 127) // 128 * 128
        import torch.distributed as dist
        from nanoplm_b200.comm.fused_optimizer import SymmetricBuffer
        g = self.group
        agreed = torch.tensor([cap], dtype=torch.int64, device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=g)
        cap = int(agreed.item())
        self._cap = cap
        self._sym = {
            "xs": SymmetricBuffer(cap * self.C, _BF16, device, g),
            "ys": SymmetricBuffer(cap * self.C, _BF16, device, g),
            "dys": SymmetricBuffer(cap * self.C, _BF16, device, g),
            "table": SymmetricBuffer(self.world * self.E, torch.int32, device, g),
            # one counter per 128-row tile of xs: rows landed since the last plan (see make_plan)
            "arrive": SymmetricBuffer(max(cap // 128, 8), torch.int32, device, g),
            # the same for the gradient rows pushed into dys, and the buffer the data gradient of the
            # dispatched rows is written to (kept apart from ys so that no barrier has to wait for the
            # peers' last reads of ys)
            "arrive_b": SymmetricBuffer(max(cap // 128, 8), torch.int32, device, g),
            "dxs": SymmetricBuffer(cap * self.C, _BF16, device, g),
            "flags": SymmetricBuffer(16, torch.int32, device, g),
        }

    def buffer(self, name: str, cap: int, device):
        """Returns (tensor [cap, C], ctypes array of the peers' base pointers). With expert
        parallelism the tensor is the layer's persistent symmetric buffer `name` (one forward /
        backward pair in flight per layer); otherwise a fresh allocation."""
        if self.world == 1:
            t = torch.empty((cap, self.C), dtype=_BF16, device=device)
            return t, _ptr_array([t.data_ptr()])
        self._ensure_symmetric(cap, device)
        sb = self._sym[name]
        return sb.tensor[: self._cap * self.C].view(self._cap, self.C), sb.ptr_array

    def table(self, device):
        if self.world == 1:
            t = torch.empty(self.E, dtype=torch.int32, device=device)
            return t, _ptr_array([t.data_ptr()])
        sb = self._sym["table"]
        return sb.tensor, sb.ptr_array

    def barrier(self, device) -> None:
        """Cross-rank flag barrier on the current stream (no-op without expert parallelism)."""
        if self.world == 1:
            return
        self.epoch += 1
        rc = lib("comm").nplm_peer_barrier(self._sym["flags"].ptr_array, c_int(self.rank), c_int(self.world),
                                           c_uint(self.epoch & 0xFFFFFFFF), c_double(self.timeout),
                                           ptr(status_word(device)), stream_ptr())
        check_rc(rc, "peer_barrier")
        count_launch()


class MoEPlan:
    """Routing plan of one forward pass (device tensors only)."""
    __slots__ = ("comm", "T", "cap", "experts", "pos_of", "group_off", "tile_group", "pad_lo", "pad_hi",
                 "tile_rows")


def make_plan(comm: MoEComm, experts: torch.Tensor) -> MoEPlan:
    """experts int32 [T,k] -> plan (counts exchange, padded offsets, row of every assignment)."""
    T, k = experts.shape
    dev = experts.device
    n = T * k
    cap = comm.capacity(n)
    if comm.world > 1:
        comm._ensure_symmetric(cap, dev)
        cap = comm._cap
    L = lib("moe")
    table, table_ptrs = comm.table(dev)
    flat = experts.reshape(-1)
    if comm.world > 1:
        # the arrival counters of this layer's dispatch start from zero: peers push only after the
        # barrier below, which this rank joins after the reset (and after everything that consumed the
        # previous dispatch) in stream order
        comm._sym["arrive"].tensor.zero_()
        comm._sym["arrive_b"].tensor.zero_()
    rc = L.nplm_moe_count(ptr(flat), c_int(n), c_int(comm.E), table_ptrs, c_int(comm.rank), c_int(comm.world),
                          stream_ptr())
    check_rc(rc, "moe_count")
    comm.barrier(dev)
    p = MoEPlan()
    p.comm, p.T, p.cap, p.experts = comm, T, cap, flat
    max_tiles = cap // 128
    p.group_off = torch.empty(comm.El + 1, dtype=torch.int32, device=dev)
    my_base = torch.empty(comm.E, dtype=torch.int32, device=dev)
    p.tile_group = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    p.pad_lo = torch.empty(comm.El, dtype=torch.int32, device=dev)
    p.pad_hi = torch.empty(comm.El, dtype=torch.int32, device=dev)
    p.tile_rows = torch.empty(max_tiles, dtype=torch.int32, device=dev) if comm.world > 1 else None
    rc = L.nplm_moe_plan(ptr(table), c_int(comm.world), c_int(comm.rank), c_int(comm.E), c_int(cap),
                         ptr(p.group_off), ptr(my_base), ptr(p.tile_group), c_int(max_tiles), ptr(p.pad_lo),
                         ptr(p.pad_hi), ptr(comm.dropped_counter(dev)), ptr(p.tile_rows), stream_ptr())
    check_rc(rc, "moe_plan")
    p.pos_of = torch.empty(n, dtype=torch.int32, device=dev)
    rc = L.nplm_moe_assign(ptr(flat), c_int(n), c_int(comm.E), ptr(my_base), ptr(p.pos_of), stream_ptr())
    check_rc(rc, "moe_assign")
    count_launch(3)
    return p


def _zero_pad(plan: MoEPlan, buf: torch.Tensor) -> None:
    c = plan.comm
    rc = lib("moe").nplm_moe_zero_pad(ptr(buf), c_int(c.C), ptr(plan.pad_lo), ptr(plan.pad_hi), c_int(c.El),
                                      c_int(plan.cap), stream_ptr())
    check_rc(rc, "moe_zero_pad")
    count_launch()


def _push(plan: MoEPlan, src, scale, dst_ptrs, arrive_ptrs=None) -> None:
    c = plan.comm
    rc = lib("moe").nplm_moe_push_rows(ptr(src), ptr(plan.experts), ptr(plan.pos_of), ptr(scale),
                                       c_int(plan.T * c.k), c_int(c.k), c_int(c.C), c_int(c.El), c_int(plan.cap),
                                       dst_ptrs, arrive_ptrs, c_int(c.world), stream_ptr())
    check_rc(rc, "moe_push_rows")
    count_launch()


def _pull(plan: MoEPlan, src_ptrs, gates) -> torch.Tensor:
    c = plan.comm
    out = torch.empty((plan.T, c.C), dtype=_BF16, device=plan.experts.device)
    rc = lib("moe").nplm_moe_pull_rows(src_ptrs, ptr(plan.experts), ptr(plan.pos_of), ptr(gates), c_int(plan.T),
                                       c_int(c.k), c_int(c.C), c_int(c.El), c_int(plan.cap), ptr(out),
                                       c_int(c.world), stream_ptr())
    check_rc(rc, "moe_pull_rows")
    count_launch()
    return out


# ------------------------------------------------------------------------------ autograd
class _RouterFn(torch.autograd.Function):
    """logits -> (gates [T,k] fp32, balance loss, experts int32 [T,k] (not differentiable))."""

    @staticmethod
    def forward(ctx, logits, k):
        probs, gates, experts, probsum, counts = router_topk(logits.contiguous(), k)
        T, E = probs.shape
        f = counts.to(torch.float32) / float(T * k)
        aux = E * (f * (probsum / T)).sum()
        ctx.save_for_backward(probs, gates, experts, f)
        ctx.mark_non_differentiable(experts)
        return gates, aux, experts

    @staticmethod
    def backward(ctx, d_gates, d_aux, _):
        probs, gates, experts, f = ctx.saved_tensors
        T, E = probs.shape
        aux_grad = None
        if d_aux is not None:
            aux_grad = (d_aux.float() * E / T * f).contiguous()
        if d_gates is None:
            d_gates = torch.zeros_like(gates)
        dlogits = router_bwd(probs, gates, experts, d_gates.float().contiguous(), aux_grad)
        return dlogits, None


class _ExpertsFn(torch.autograd.Function):
    """y[t] = sum_s gates[t,s] * Expert_{e(t,s)}(x[t]) with SwiGLU experts, all on the device:
    push rows -> grouped up-projection (+SwiGLU) -> grouped down-projection -> weighted pull.
    Barriers (expert parallelism only) separate the phases that touch peers' buffers."""

    @staticmethod
    def forward(ctx, x, gates, Wi, Wo, plan):
        c = plan.comm
        dev = x.device
        ep = c.world > 1
        xs, xs_ptrs = c.buffer("xs", plan.cap, dev)
        _zero_pad(plan, xs)
        pre = torch.empty((plan.cap, Wi.shape[1]), dtype=_BF16, device=dev)
        if ep and c.gated_dispatch:
            # no barrier between dispatch and up-projection: every pushed row bumps the arrival counter of
            # its tile on the owner, and the grouped GEMM loads a tile once its rows have landed
            arrive = c._sym["arrive"]
            _push(plan, x.contiguous(), None, xs_ptrs, arrive.ptr_array)
            h = gemm_grouped(xs, Wi, plan.tile_group, epi=K.EPI_SWIGLU, aux=pre,
                             arrive=arrive.tensor, expect=plan.tile_rows)
        else:
            _push(plan, x.contiguous(), None, xs_ptrs)
            c.barrier(dev)                                # all rows of my experts have arrived
            h = gemm_grouped(xs, Wi, plan.tile_group, epi=K.EPI_SWIGLU, aux=pre)
        ys, ys_ptrs = c.buffer("ys", plan.cap, dev)
        gemm_grouped(h, Wo, plan.tile_group, out=ys)
        c.barrier(dev)                                    # every owner's outputs are complete
        gates32 = gates.float().contiguous()
        y = _pull(plan, ys_ptrs, gates32)
        ctx.plan = plan
        if ep:
            ctx.save_for_backward(gates32, Wi, Wo, pre, h)
        else:
            ctx.save_for_backward(gates32, Wi, Wo, pre, h, xs, ys)
        ctx.Wi_ref, ctx.Wo_ref = Wi, Wo
        return y

    @staticmethod
    def backward(ctx, dy):
        from .functional import _has_main_grad
        plan = ctx.plan
        c = plan.comm
        dev = dy.device
        ep = c.world > 1
        if ep:
            gates32, Wi, Wo, pre, h = ctx.saved_tensors
            xs, xs_ptrs = c.buffer("xs", plan.cap, dev)    # still holds this layer's forward rows
            ys, ys_ptrs = c.buffer("ys", plan.cap, dev)
        else:
            gates32, Wi, Wo, pre, h, xs, ys = ctx.saved_tensors
            ys_ptrs = _ptr_array([ys.data_ptr()])
        n = plan.T * c.k
        dy = dy.contiguous()
        # gradient of combine: d_gates = <dy, ys row> (pulled), d_ys = gate * dy (pushed to the owner)
        dys, dys_ptrs = c.buffer("dys", plan.cap, dev)
        _zero_pad(plan, dys)
        d_gates = torch.empty((plan.T, c.k), dtype=torch.float32, device=dev)
        gated = ep and c.gated_backward
        arrive_b = c._sym["arrive_b"] if gated else None
        rc = lib("moe").nplm_moe_combine_bwd(ptr(dy), ys_ptrs, dys_ptrs, ptr(plan.experts), ptr(plan.pos_of),
                                             ptr(gates32), c_int(n), c_int(c.k), c_int(c.C), c_int(c.El),
                                             c_int(plan.cap), ptr(d_gates),
                                             arrive_b.ptr_array if gated else None, c_int(c.world), stream_ptr())
        check_rc(rc, "moe_combine_bwd")
        count_launch()
        if gated:
            # no barrier: the down-projection's data gradient starts tile by tile as the d_ys rows land,
            # and the data gradient of the dispatched rows goes to a buffer of its own (peers may still
            # be reading ys)
            d_h = gemm_grouped(dys, Wo, plan.tile_group, b_mn=True, arrive=arrive_b.tensor, expect=plan.tile_rows)
            dxs, dx_ptrs = c.buffer("dxs", plan.cap, dev)
        else:
            c.barrier(dev)                                # d_ys complete, nobody reads ys any more
            d_h = gemm_grouped(dys, Wo, plan.tile_group, b_mn=True)
            # the data gradient of the dispatched rows lands in the buffer that held ys
            dxs, dx_ptrs = (ys, ys_ptrs) if ep else (None, None)
        d_pre = K.swiglu_bwd(pre, d_h)
        dxs = gemm_grouped(d_pre, Wi, plan.tile_group, b_mn=True, out=dxs)
        if not ep:
            dx_ptrs = _ptr_array([dxs.data_ptr()])
        Wi_p, Wo_p = ctx.Wi_ref, ctx.Wo_ref
        gWi = gWo = None
        if _has_main_grad(Wo_p):
            gemm_grouped_wgrad(dys, h, plan.group_off, Wo_p.main_grad.view(Wo.shape))
        else:
            acc = torch.zeros(Wo.shape, dtype=torch.float32, device=dev)
            gWo = gemm_grouped_wgrad(dys, h, plan.group_off, acc).to(Wo.dtype)
        if _has_main_grad(Wi_p):
            gemm_grouped_wgrad(d_pre, xs, plan.group_off, Wi_p.main_grad.view(Wi.shape))
        else:
            acc = torch.zeros(Wi.shape, dtype=torch.float32, device=dev)
            gWi = gemm_grouped_wgrad(d_pre, xs, plan.group_off, acc).to(Wi.dtype)
        c.barrier(dev)                                    # every owner's d_xs is complete
        dx = _pull(plan, dx_ptrs, None)
        if not gated:
            c.barrier(dev)                                # peers are done reading before buffers are reused
        # (gated: the next write into any of this layer's buffers by a peer or by this rank comes after
        # the barrier of the next make_plan, which every rank joins after this pull in stream order)
        return dx, d_gates, gWi, gWo, None


def moe_mlp(x: torch.Tensor, router_logits: torch.Tensor, Wi: torch.Tensor, Wo: torch.Tensor, top_k: int,
            comm: MoEComm):
    """Full MoE MLP on the device path. x bf16 [T,C]; router_logits bf16 [T,E]; Wi [El, 2I, C];
    Wo [El, C, I]. Returns (y [T,C], aux loss scalar fp32)."""
    gates, aux, experts = _RouterFn.apply(router_logits, top_k)
    plan = make_plan(comm, experts)
    y = _ExpertsFn.apply(x, gates, Wi, Wo, plan)
    return y, aux
