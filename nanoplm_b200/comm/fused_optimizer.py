"""Optimizer step with the collectives fused into the kernels (reduce-scatter + gradient norm,
AdamW + all-gather push) over symmetric memory. See nanoplm_b200/csrc/comm.cu.

The reduce-scatter is split by parameter and overlapped with the backward pass of the last
micro-step, as the reference's FSDP2 does with its per-layer reduce-scatter
(src/nanoplm/pretraining/pure_pipeline.py:697-702, 736-742): when the weight-gradient GEMM of a
parameter has been launched (`ops.functional.set_wgrad_ready_callback`), a side stream waits for that
GEMM, passes a peer barrier of its own (every rank's gradient of this parameter is final) and the
owner(s) of the parameter's slice pull and sum it while the main stream continues with the next
layer's backward. After the backward pass only the parameters without such a GEMM (embedding,
norms, head) and the parameter that finished last remain, then the norm exchange and the
AdamW + push.

`FusedShardedStep.try_create` allocates the gradient buffer, the parameter buffer and the flag /
slot words in symmetric memory (torch.distributed._symmetric_memory: CUDA VMM allocations whose
handles are exchanged once over the bootstrap process group and mapped into every rank). If that
is not possible on the machine (no peer access, more than 8 ranks, symmetric memory unavailable) it
returns None and the engine keeps using NCCL collectives.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist

from nanoplm_b200.ops._lib import check_rc, count_launch, lib, ptr, status_word, stream_ptr
from nanoplm_b200.utils.logging import logger

MAX_PEERS = 8


def _ptr_array(ptrs):
    arr = (c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = c_void_p(int(p))
    return arr


class SymmetricBuffer:
    """A tensor allocated identically on every rank, with the peers' device addresses."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group):
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ptr_array = _ptr_array(self.ptrs)


class FusedShardedStep:
    def __init__(self, engine, grads: SymmetricBuffer, params: SymmetricBuffer, words: SymmetricBuffer,
                 barrier_timeout_s: float = 20.0):
        self.e = engine
        self.grads, self.params, self.words = grads, params, words
        self.world, self.rank = engine.world, engine.rank
        self.epoch = 0
        self.timeout = barrier_timeout_s
        dev = engine.device
        self.shard_grad = torch.zeros(engine.shard, dtype=torch.float32, device=dev)
        self.partial = torch.zeros(1, dtype=torch.float32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        # words layout per rank: [0:8] barrier flags (uint32), [8:16] partial sums (float32 bits)
        self.flag_ptrs = _ptr_array(words.ptrs)
        self.slot_ptrs = _ptr_array([p + 8 * 4 for p in words.ptrs])
        self.local_slots = words.tensor.view(torch.float32)[8:16]
        # [16:24]: flags of the side-stream barriers (one per overlapped parameter, own epoch counter)
        self.side_flag_ptrs = _ptr_array([p + 16 * 4 for p in words.ptrs])
        self.side_epoch = 0
        self.side_stream = torch.cuda.Stream(dev)
        self._lib = lib("comm")
        # ranges [a, b) of the owned slice that were reduced during the backward pass of this step
        self.done: list[tuple[int, int]] = []
        self.armed = False
        self.overlapped_bytes = 0
        self._events: list[torch.cuda.Event] = []
        # CUDA events bracketing the part of step() that runs after the backward pass (not overlapped)
        self.timing = False
        self.tail_events: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []

    # ------------------------------------------------------------------ construction
    @staticmethod
    def allocate(total: int, world: int, device: torch.device, group, compute_dtype):
        """Returns (grads, params, words) symmetric buffers or None when unavailable."""
        if world > MAX_PEERS or compute_dtype != torch.bfloat16:
            return None
        try:
            g = group if group is not None else dist.group.WORLD
            grads = SymmetricBuffer(total, torch.float32, device, g)
            params = SymmetricBuffer(total, torch.bfloat16, device, g)
            words = SymmetricBuffer(32, torch.int32, device, g)
            ok = torch.ones(1, device=device)
        except Exception as exc:  # noqa: BLE001
            logger.warning(f"symmetric memory unavailable ({type(exc).__name__}: {exc}); using NCCL collectives")
            ok = torch.zeros(1, device=device)
            grads = params = words = None
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if ok.item() < 1:
            return None
        return grads, params, words

    # ------------------------------------------------------------------ step
    def barrier(self) -> None:
        self.epoch += 1
        rc = self._lib.nplm_peer_barrier(self.flag_ptrs, c_int(self.rank), c_int(self.world),
                                         c_uint(self.epoch & 0xFFFFFFFF), c_double(self.timeout),
                                         ptr(status_word(self.e.device)), stream_ptr())
        check_rc(rc, "peer_barrier")
        count_launch()

    # ------------------------------------------------------------------ overlap with backward
    def arm(self) -> None:
        """Call before the forward pass of the LAST micro-step of an optimizer step (on every rank):
        from now on a parameter whose weight-gradient kernel has been launched is final."""
        self.armed = True
        self.done = []
        self.partial.zero_()
        self.overlapped_bytes = 0

    def _rs(self, a: int, b: int) -> None:
        """Sums [a, b) (global flat indices inside the owned slice) over all ranks on the current stream."""
        e = self.e
        rc = self._lib.nplm_rs_sumsq(self.grads.ptr_array, c_int(self.world), c_longlong(a), c_longlong(b - a),
                                     c_void_p(self.shard_grad.data_ptr() + 4 * (a - e.lo)), ptr(self.partial),
                                     stream_ptr())
        check_rc(rc, "rs_sumsq")
        count_launch()

    def on_wgrad_ready(self, slot_range: tuple[int, int]) -> None:
        """Side stream: wait for the gradient kernel just launched, barrier with the peers, reduce the
        part of [offset, offset + numel) this rank owns."""
        if not self.armed:
            return
        e = self.e
        lo, hi = slot_range
        if (lo | hi) & 7:                                 # odd-sized tensor: left to the final pass
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(e.device))
        self._events.append(ev)
        with torch.cuda.stream(self.side_stream):
            self.side_stream.wait_event(ev)
            self.side_epoch += 1
            rc = self._lib.nplm_peer_barrier(self.side_flag_ptrs, c_int(self.rank), c_int(self.world),
                                             c_uint(self.side_epoch & 0xFFFFFFFF), c_double(self.timeout),
                                             ptr(status_word(e.device)), stream_ptr())
            check_rc(rc, "peer_barrier")
            count_launch()
            a, b = max(lo, e.lo), min(hi, e.hi)
            if b > a:
                self._rs(a, b)
                self.done.append((a, b))
                self.overlapped_bytes += 4 * (b - a) * self.world

    def _remaining(self) -> list[tuple[int, int]]:
        e = self.e
        out, cur = [], e.lo
        for a, b in sorted(self.done):
            if a > cur:
                out.append((cur, a))
            cur = max(cur, b)
        if cur < e.hi:
            out.append((cur, e.hi))
        return out

    def step(self, lr: float, grad_scale: float, extra_sumsq=None) -> torch.Tensor:
        """extra_sumsq: sum of squares (already summed over the ranks, same scaling) of gradients held
        outside the flat buffer (expert weights); it enters the clipping norm through rank 0's partial
        sum, and the engine's `_sumsq` receives the global sum for those parameters' own update."""
        e = self.e
        main = torch.cuda.current_stream(e.device)
        if self.timing:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(main)
        if not self.armed:
            self.done = []
            self.partial.zero_()
        else:
            main.wait_stream(self.side_stream)           # the overlapped reductions have finished
        self.armed = False
        self._events = []
        self.barrier()                                   # every rank's gradients are final
        for a, b in self._remaining():
            self._rs(a, b)
        if extra_sumsq is not None and self.rank == 0:
            self.partial += extra_sumsq.to(torch.float32).reshape(1)
        rc = self._lib.nplm_publish(self.slot_ptrs, c_int(self.rank), c_int(self.world), ptr(self.partial),
                                    stream_ptr())
        check_rc(rc, "publish")
        self.barrier()                                   # partial sums exchanged, peers done reading my gradients
        e.main_grad.zero_()
        rc = self._lib.nplm_adamw_push(ptr(e.master), ptr(e.exp_avg), ptr(e.exp_avg_sq), ptr(self.shard_grad),
                                       self.params.ptr_array, c_int(self.world), c_longlong(e.lo),
                                       c_longlong(e.shard), c_longlong(e.decay_end), ptr(e._hyper_dev[0]),
                                       ptr(self.local_slots), ptr(self.norm), stream_ptr())
        check_rc(rc, "adamw_push")
        count_launch(2)
        self.barrier()                                   # every rank's parameter buffer is complete
        if extra_sumsq is not None:
            e._sumsq.copy_((self.norm / grad_scale) ** 2)
        if self.timing:
            t1.record(main)
            self.tail_events.append((t0, t1))
        return self.norm[0]


class ParamShardedStep(FusedShardedStep):
    """Optimizer step of `ParamShardedEngine`: the same kernels on row-block ownership. Every rank
    reduces its own row block of a matrix as soon as that matrix's gradient kernel of the last
    micro-step has been launched (so the reduction work of every parameter is spread over all ranks
    and hidden under the backward pass), AdamW updates the owned rows in place, and nothing is
    pushed for matrices the next forward pass gathers inside its GEMMs."""

    def __init__(self, engine, grads, params, words, barrier_timeout_s: float = 20.0):
        super().__init__(engine, grads, params, words, barrier_timeout_s)
        self.self_ptr = _ptr_array([params.ptrs[self.rank]])
        self.by_offset = {p.slot.offset: p for p in engine.mine}
        self.done_ids: set[int] = set()

    def arm(self) -> None:
        super().arm()
        self.done_ids = set()

    def _rs_piece(self, p) -> None:
        rc = self._lib.nplm_rs_sumsq(self.grads.ptr_array, c_int(self.world), c_longlong(p.a),
                                     c_longlong(p.b - p.a), c_void_p(self.shard_grad.data_ptr() + 4 * p.local),
                                     ptr(self.partial), stream_ptr())
        check_rc(rc, "rs_sumsq")
        count_launch()

    def on_wgrad_ready(self, slot_range: tuple[int, int]) -> None:
        if not self.armed:
            return
        e = self.e
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(e.device))
        self._events.append(ev)
        with torch.cuda.stream(self.side_stream):
            self.side_stream.wait_event(ev)
            self.side_epoch += 1
            rc = self._lib.nplm_peer_barrier(self.side_flag_ptrs, c_int(self.rank), c_int(self.world),
                                             c_uint(self.side_epoch & 0xFFFFFFFF), c_double(self.timeout),
                                             ptr(status_word(e.device)), stream_ptr())
            check_rc(rc, "peer_barrier")
            count_launch()
            p = self.by_offset.get(slot_range[0])
            if p is not None and id(p) not in self.done_ids:
                self._rs_piece(p)
                self.done_ids.add(id(p))
                self.overlapped_bytes += 4 * (p.b - p.a) * self.world

    def step(self, lr: float, grad_scale: float) -> torch.Tensor:
        e = self.e
        main = torch.cuda.current_stream(e.device)
        if self.timing:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(main)
        if not self.armed:
            self.done_ids = set()
            self.partial.zero_()
        else:
            main.wait_stream(self.side_stream)
        self.armed = False
        self._events = []
        self.barrier()                                   # every rank's gradients are final
        for p in e.mine:
            if id(p) not in self.done_ids:
                self._rs_piece(p)
        rc = self._lib.nplm_publish(self.slot_ptrs, c_int(self.rank), c_int(self.world), ptr(self.partial),
                                    stream_ptr())
        check_rc(rc, "publish")
        self.barrier()                                   # partial sums exchanged, peers done reading my gradients
        e.main_grad.zero_()
        f4 = 4
        for p in e.mine:
            loc = f4 * p.local
            # gathered row blocks stay local (the consuming GEMM of the next forward pass fetches them);
            # the small tensors go to every rank
            ptrs, push_world = (self.self_ptr, 1) if p.gathered else (self.params.ptr_array, self.world)
            rc = self._lib.nplm_adamw_push_ex(
                c_void_p(e.master.data_ptr() + loc), c_void_p(e.exp_avg.data_ptr() + loc),
                c_void_p(e.exp_avg_sq.data_ptr() + loc), c_void_p(self.shard_grad.data_ptr() + loc), ptrs,
                c_int(push_world), c_longlong(p.a), c_longlong(p.b - p.a), c_longlong(e.decay_end),
                ptr(e._hyper_dev[0]), ptr(self.local_slots), c_int(self.world), ptr(self.norm), stream_ptr())
            check_rc(rc, "adamw_push")
        count_launch(1 + len(e.mine))
        self.barrier()                                   # every rank's rows are final before anybody gathers them
        if self.timing:
            t1.record(main)
            self.tail_events.append((t0, t1))
        return self.norm[0]


class MuonPeerStep:
    """Peer-memory communication of the Muon / NorMuon step (`parallel.muon.MuonEngine`), replacing the
    all-reduce of the whole fp32 gradient and the all-gathers of the orthogonalised updates:

    * every matrix has one owner rank (the rank that orthogonalises it): the owner PULLS and sums the
      matrix's gradient from all ranks (`rs_sumsq_kernel`, rank order), nobody else reads it;
    * the few tensors AdamW updates on every rank (embedding, norms, head) are summed by every rank in the
      same fixed order, so the replicas stay bitwise equal;
    * the squared norm for clipping: per-rank partial sums (rank 0 adds the AdamW tensors' share) are
      exchanged through the slot words and added in rank order on every rank;
    * the owner stores its orthogonalised updates straight into every peer's copy of the stack buffer
      (`push_kernel`); one flag barrier later every rank applies all updates locally.
    """

    def __init__(self, engine, grads: SymmetricBuffer, params: SymmetricBuffer, words: SymmetricBuffer,
                 barrier_timeout_s: float = 20.0):
        self.e = engine
        self.grads, self.params, self.words = grads, params, words
        self.world, self.rank = engine.world, engine.rank
        self.epoch = 0
        self.timeout = barrier_timeout_s
        dev = engine.device
        self.partial = torch.zeros(1, dtype=torch.float32, device=dev)
        self.adam_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.flag_ptrs = _ptr_array(words.ptrs)
        self.slot_ptrs = _ptr_array([p + 8 * 4 for p in words.ptrs])
        self.local_slots = words.tensor.view(torch.float32)[8:16]
        self._lib = lib("comm")
        self.reduced = None            # full-size fp32 buffer holding the sums this rank needs
        self.stack_buffers: list[SymmetricBuffer] = []
        self.adam_ranges: list[tuple[int, int]] = []
        self.nvlink_bytes_in = 0

    barrier = FusedShardedStep.barrier

    def arm(self) -> None:             # the reduction is not split over the backward pass here
        pass

    def setup(self, stacks, adam_slots) -> None:
        """Collective: allocates one symmetric bf16 buffer per stack of same-shape matrices."""
        e = self.e
        g = e.pg if e.pg is not None else dist.group.WORLD
        for st in stacks:
            self.stack_buffers.append(SymmetricBuffer(len(st.slots) * st.slots[0].numel, torch.bfloat16, e.device, g))
        self.reduced = torch.zeros(e.total, dtype=torch.float32, device=e.device)
        # contiguous runs of AdamW tensors (slot starts are 64-element aligned, the gaps hold zeros)
        spans = sorted((s.offset, s.offset + ((s.numel + 3) // 4) * 4) for s in adam_slots)
        for a, b in spans:
            if self.adam_ranges and a <= self.adam_ranges[-1][1] + 64:
                self.adam_ranges[-1] = (self.adam_ranges[-1][0], max(b, self.adam_ranges[-1][1]))
            else:
                self.adam_ranges.append((a, b))

    def _rs(self, a: int, b: int, sumsq: torch.Tensor) -> None:
        rc = self._lib.nplm_rs_sumsq(self.grads.ptr_array, c_int(self.world), c_longlong(a), c_longlong(b - a),
                                     c_void_p(self.reduced.data_ptr() + 4 * a), ptr(sumsq), stream_ptr())
        check_rc(rc, "rs_sumsq")
        count_launch()

    def reduce(self, owned_slots, gsq: torch.Tensor) -> torch.Tensor:
        """Fills `reduced` with the summed gradients of this rank's matrices and of the AdamW tensors,
        `gsq` with the squared norm of the whole summed gradient; returns `reduced`."""
        self.barrier()                                   # every rank's gradients are final
        self.partial.zero_()
        self.adam_sq.zero_()
        n = 0
        for s in owned_slots:
            self._rs(s.offset, s.offset + s.numel, self.partial)
            n += s.numel
        for a, b in self.adam_ranges:
            self._rs(a, b, self.adam_sq)
            n += b - a
        self.nvlink_bytes_in = 4 * n * (self.world - 1)
        if self.rank == 0:
            self.partial += self.adam_sq
        rc = self._lib.nplm_publish(self.slot_ptrs, c_int(self.rank), c_int(self.world), ptr(self.partial),
                                    stream_ptr())
        check_rc(rc, "publish")
        count_launch()
        self.barrier()                                   # partial sums exchanged
        gsq.zero_()
        for r in range(self.world):                      # same order on every rank: identical clip coefficient
            gsq += self.local_slots[r:r + 1]
        return self.reduced

    def push_run(self, index: int, first: int, count: int, numel: int) -> None:
        """Stores matrices [first, first + count) of stack `index` into every peer's stack buffer."""
        if count <= 0:
            return
        buf = self.stack_buffers[index]
        rc = self._lib.nplm_push(buf.ptr_array, c_int(self.rank), c_int(self.world), c_longlong(2 * first * numel),
                                 c_longlong(2 * count * numel), stream_ptr())
        check_rc(rc, "push")
        count_launch()
