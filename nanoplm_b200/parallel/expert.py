"""Expert parallelism: the experts of a MoE layer are split over the ranks of a process group; rows
(tokens already sorted by global expert id) are exchanged with an all-to-all before the expert
GEMMs and returned with a second all-to-all.

This is the collective-library version (NCCL `all_to_all_single`; an all-gather based emulation on
gloo so the routing tables can be tested on CPU ranks). Row counts are exchanged first so every
rank knows how many rows each peer sends for each of its local experts.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _all_to_all_rows(rows: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    out = torch.empty((sum(recv_counts), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    if rows.is_cuda:
        dist.all_to_all_single(out, rows.contiguous(), recv_counts, send_counts, group=group)
        return out
    # gloo: gather everything, then pick the slices addressed to this rank
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    sizes = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor(send_counts, dtype=torch.int64), group=group)
    max_rows = int(max(int(s.sum()) for s in sizes))
    pad = torch.zeros((max_rows, rows.shape[1]), dtype=rows.dtype)
    pad[:rows.shape[0]] = rows
    bufs = [torch.zeros_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    parts = []
    for src in range(world):
        start = int(sizes[src][:rank].sum())
        parts.append(bufs[src][start:start + int(sizes[src][rank])])
    return torch.cat(parts, dim=0)


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, send_counts, recv_counts, group):
        ctx.cfg = (send_counts, recv_counts, group)
        return _all_to_all_rows(rows, send_counts, recv_counts, group)

    @staticmethod
    def backward(ctx, d):
        send_counts, recv_counts, group = ctx.cfg
        return _all_to_all_rows(d.contiguous(), recv_counts, send_counts, group), None, None, None


def expert_parallel_apply(moe, rows: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """rows: [T*k, C] sorted by global expert; counts: [E] rows per global expert (this rank's tokens).
    Returns the expert outputs in the same row order."""
    group, world = moe.ep_group, moe.ep_world
    L = moe.local_experts
    # counts_all[src][e]: rows rank `src` holds for global expert e
    counts_all = [torch.zeros_like(counts) for _ in range(world)]
    dist.all_gather(counts_all, counts, group=group)
    counts_all = torch.stack(counts_all).cpu()                     # [world, E]
    mine = counts_all[moe.ep_rank]
    send_counts = [int(mine[d * L:(d + 1) * L].sum()) for d in range(world)]
    lo, hi = moe.ep_rank * L, (moe.ep_rank + 1) * L
    recv_counts = [int(counts_all[s, lo:hi].sum()) for s in range(world)]
    recv = _AllToAll.apply(rows, send_counts, recv_counts, group)
    # received rows are ordered (source rank, local expert); regroup by local expert
    per = counts_all[:, lo:hi]                                    # [world, L]
    idx, offs, base = [], [], 0
    for s in range(world):
        start = base
        for e in range(L):
            n = int(per[s, e])
            offs.append((e, s, start, n))
            start += n
        base += recv_counts[s]
    order = []
    for e in range(L):
        for (ee, s, start, n) in offs:
            if ee == e and n:
                order.append(torch.arange(start, start + n))
    if order:
        perm = torch.cat(order).to(rows.device)
    else:
        perm = torch.zeros(0, dtype=torch.long, device=rows.device)
    grouped = recv[perm]
    out = moe._run_experts(grouped, [int(per[:, e].sum()) for e in range(L)])
    back = torch.empty_like(out)
    back[perm] = out
    return _AllToAll.apply(back, recv_counts, send_counts, group)
