"""All-reduce of a handful of host statistics (token counts, elapsed time, ...) in one kernel over
peer memory (nanoplm_b200/csrc/comm.cu: stats_allreduce_kernel).

The reference reduces these with separate NCCL calls at every logging boundary: SUM of tokens, SUM
of raw tokens, MAX of the elapsed time (src/nanoplm/pretraining/pure_pipeline.py:775-800). Here the
ranks exchange up to 16 doubles through a table in symmetric memory; each value is summed or
maximised according to a bit mask. Waits are bounded: a peer that never arrives raises
`CommTimeout` and leaves the CUDA context usable.
"""
from __future__ import annotations

from ctypes import c_double, c_int, c_uint

import torch
import torch.distributed as dist

from nanoplm_b200.ops._lib import check_rc, check_status, count_launch, lib, ptr, status_word, stream_ptr
from nanoplm_b200.utils.logging import logger

MAX_VALUES = 16


class PeerStats:
    def __init__(self, device: torch.device, rank: int, world: int, ptr_array, keepalive, timeout_s: float = 20.0):
        self.device, self.rank, self.world = device, rank, world
        self.ptr_array, self._keepalive = ptr_array, keepalive
        self.timeout = timeout_s
        self.epoch = 0
        self._in = torch.zeros(MAX_VALUES, dtype=torch.float64, device=device)
        self._out = torch.zeros(MAX_VALUES, dtype=torch.float64, device=device)
        self._lib = lib("comm")

    @staticmethod
    def try_create(device: torch.device, group=None, timeout_s: float = 20.0):
        """Collective. Returns a PeerStats, or None when symmetric memory cannot be set up on every
        rank (the caller then keeps using library all-reduces). A single process gets a table in
        ordinary device memory."""
        from nanoplm_b200.comm.fused_optimizer import MAX_PEERS, SymmetricBuffer, _ptr_array
        nbytes = int(lib("comm").nplm_stats_buffer_bytes())
        words = (nbytes + 3) // 4
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            buf = torch.zeros(words, dtype=torch.int32, device=device)
            return PeerStats(device, 0, 1, _ptr_array([buf.data_ptr()]), buf, timeout_s)
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ok = torch.ones(1, device=device)
        sym = None
        if world > MAX_PEERS:
            ok.zero_()
        else:
            try:
                sym = SymmetricBuffer(words, torch.int32, device, group if group is not None else dist.group.WORLD)
            except Exception as exc:  # noqa: BLE001
                logger.warning(f"symmetric memory unavailable for the statistics table ({type(exc).__name__}: {exc})")
                ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() < 1:
            return None
        return PeerStats(device, rank, world, sym.ptr_array, sym, timeout_s)

    def all_reduce(self, values, max_mask: int = 0) -> list:
        """values: up to 16 numbers of this rank. Returns the reduced list (bit i of max_mask set:
        maximum of value i over the ranks, else the sum). Synchronises the stream (host result)."""
        n = len(values)
        if not 1 <= n <= MAX_VALUES:
            raise ValueError(f"between 1 and {MAX_VALUES} values, got {n}")
        self._in[:n].copy_(torch.tensor(list(values), dtype=torch.float64), non_blocking=False)
        self.epoch = self.epoch % 0x7FFFFFFF + 1
        rc = self._lib.nplm_stats_allreduce(self.ptr_array, c_int(self.rank), c_int(self.world), c_uint(self.epoch),
                                            ptr(self._in), ptr(self._out), c_int(n), c_uint(max_mask),
                                            c_double(self.timeout), ptr(status_word(self.device)), stream_ptr())
        check_rc(rc, "stats_allreduce")
        count_launch()
        out = self._out[:n].tolist()
        check_status(self.device)
        return out
