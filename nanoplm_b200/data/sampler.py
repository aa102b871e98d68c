"""Length-aware batching for data-parallel training on packed batches.

With the padding tail of a packed micro-batch cut off, the work of a micro-batch is no longer a
constant: it follows the real tokens (and, in full-attention layers, the squared sequence lengths)
it happens to hold. Every optimizer step ends in a collective, so the step takes as long as the
slowest rank; with two micro-batches per rank the spread is a few per cent of the step. The
reference pads every micro-batch to one static shape (src/nanoplm/pretraining/collator.py:405-458),
which hides the effect by doing the maximum work everywhere.

`BalancedBatchSampler` keeps the global batch of an optimizer step exactly what a shuffled sampler
would have produced (the next `micro_batch_size x grad_accum x world` indices of the epoch's
permutation), but deals those sequences to the (rank, micro-step) bins with
`nanoplm_b200.data.packing.balance_bins`, so every bin holds the same number of sequences and
(nearly) the same cost. Every rank computes the same assignment and keeps its own bins.
"""
from __future__ import annotations

from typing import Iterator, Optional

import numpy as np
import torch
from torch.utils.data import Sampler

from .packing import DEFAULT_QUADRATIC_COST, balance_bins


class BalancedBatchSampler(Sampler):
    """Batch sampler: yields this rank's micro-batches (lists of dataset indices), `grad_accum` per
    optimizer step. A trailing window that does not fill a whole optimizer step is dropped.
    `fast_forward(n)` skips the first n micro-batches of the next epoch in O(1)."""

    def __init__(self, lengths, micro_batch_size: int, grad_accum: int, world: int = 1, rank: int = 0,
                 shuffle: bool = True, seed: int = 0, quad: float = DEFAULT_QUADRATIC_COST,
                 max_length: Optional[int] = None):
        self.lengths = np.asarray(lengths, dtype=np.int32)
        if max_length is not None:
            self.lengths = np.minimum(self.lengths, int(max_length))
        self.mbs, self.accum, self.world, self.rank = int(micro_batch_size), int(grad_accum), int(world), int(rank)
        self.shuffle, self.seed, self.quad = shuffle, seed, float(quad)
        self.window = self.mbs * self.accum * self.world
        self.steps = len(self.lengths) // self.window
        self.epoch, self.start_micro = 0, 0
        self.last_costs: Optional[np.ndarray] = None     # bin costs of the last step dealt (all ranks)

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def fast_forward(self, micro_batches: int) -> None:
        self.start_micro = max(0, min(self.steps * self.accum, int(micro_batches)))

    def __len__(self) -> int:
        return self.steps * self.accum - self.start_micro

    def step_bins(self, order: np.ndarray, step: int) -> list[np.ndarray]:
        """All (rank, micro-step) bins of optimizer step `step`: bin a * world + r is micro-step a of rank r."""
        win = order[step * self.window:(step + 1) * self.window]
        bin_of, cost = balance_bins(self.lengths[win], self.accum * self.world, self.mbs, self.quad)
        self.last_costs = cost
        return [win[bin_of == b] for b in range(self.accum * self.world)]

    def __iter__(self) -> Iterator[list[int]]:
        n = len(self.lengths)
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch)
            order = torch.randperm(n, generator=g).numpy()
        else:
            order = np.arange(n)
        start, self.start_micro = self.start_micro, 0
        for step in range(start // self.accum, self.steps):
            bins = self.step_bins(order, step)
            for a in range(self.accum):
                if step * self.accum + a < start:
                    continue
                yield bins[a * self.world + self.rank].tolist()
