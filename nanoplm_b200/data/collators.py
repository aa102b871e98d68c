"""Batch collators for MLM pretraining.

`ProtDataCollatorForLM` pads to the longest sequence of the batch; `PackingCollator` packs
sequences into rows (dynamic 2-D output) or into the flat static layout. Output keys, dtypes and
semantics match the reference collators (src/nanoplm/pretraining/collator.py:7-458); packing and
masking run in C++ / vectorised numpy instead of per-row Python loops.

Both add two keys the native trainer uses and the reference ignores: `masked_idx` (int32 indices of
the positions with a label, into the flat token axis) and `masked_labels` (their labels), so the
MLM head only runs on masked positions.
"""
from __future__ import annotations

from typing import Iterable, Optional, Sequence

import numpy as np
import torch

from .masking import MLMMasker
from .packing import flatten, pack_ffd, static_cu_seqlens


def _example_ids(ex) -> np.ndarray:
    ids = ex["input_ids"]
    if isinstance(ids, torch.Tensor):
        ids = ids.numpy()
    ids = np.asarray(ids)
    mask = ex.get("attention_mask") if isinstance(ex, dict) else None
    if mask is not None:
        if isinstance(mask, torch.Tensor):
            mask = mask.numpy()
        ids = ids[: int(np.asarray(mask).sum())]
    return ids.astype(np.uint8, copy=False)


class _CollatorBase:
    def __init__(self, tokenizer, mlm_probability, mask_token_probability, random_token_probability,
                 keep_probability, extra_excluded_token_ids, seed):
        self.tokenizer = tokenizer
        self.mlm_probability = mlm_probability
        self.masker = MLMMasker(tokenizer, mlm_probability, mask_token_probability,
                                random_token_probability, keep_probability, extra_excluded_token_ids)
        self.p_mask, self.p_rand, self.p_keep = self.masker.p_mask, self.masker.p_rand, self.masker.p_keep
        self.allowed_random_token_ids = torch.from_numpy(self.masker.allowed_random_token_ids)
        self.pad_token_id = getattr(tokenizer, "pad_token_id", 0) or 0
        self._seed = seed
        self._rng: np.random.Generator | None = None

    def rng(self) -> np.random.Generator:
        # created lazily so every DataLoader worker process gets its own stream
        if self._rng is None:
            seed = self._seed
            info = torch.utils.data.get_worker_info()
            if seed is None:
                seed = int(torch.initial_seed() % (2 ** 63))
            elif info is not None:
                seed = seed + 7919 * (info.id + 1)
            self._rng = np.random.default_rng(seed)
        return self._rng

    def reseed(self, seed: int) -> None:
        self._seed, self._rng = seed, None


class ProtDataCollatorForLM(_CollatorBase):
    """Padded MLM batches: input_ids / attention_mask / labels of shape (B, max_len_in_batch)."""

    def __init__(self, tokenizer, mlm_probability: float = 0.03, mask_token_probability: float = 0.80,
                 random_token_probability: float = 0.10, keep_probability: float = 0.10, *,
                 extra_excluded_token_ids: Optional[Iterable[int]] = None, seed: int | None = None):
        super().__init__(tokenizer, mlm_probability, mask_token_probability, random_token_probability,
                         keep_probability, extra_excluded_token_ids, seed)

    def __call__(self, examples: Sequence[dict]) -> dict:
        seqs = [_example_ids(e) for e in examples]
        width = max((len(s) for s in seqs), default=0)
        ids = np.full((len(seqs), width), self.pad_token_id, dtype=np.int64)
        att = np.zeros((len(seqs), width), dtype=np.int64)
        for i, s in enumerate(seqs):
            ids[i, :len(s)] = s
            att[i, :len(s)] = 1
        new_ids, labels = self.masker(ids, self.rng(), forbid=att == 0)
        return {"input_ids": torch.from_numpy(new_ids), "attention_mask": torch.from_numpy(att),
                "labels": torch.from_numpy(labels)}


class PackingCollator(_CollatorBase):
    """First-fit-decreasing packing + MLM masking.

    Dynamic mode (target_rows None): input_ids / attention_mask / labels (R, W), cu_seqlens (N+1,)
    int32, max_seqlen int.  Static mode: 1-D input_ids / labels / position_ids of length
    F = target_rows * W, cu_seqlens of fixed length batch_size + 1 + target_rows, max_seqlen = W.
    """

    def __init__(self, tokenizer, max_seq_len: int, mlm_probability: float = 0.03,
                 mask_token_probability: float = 0.80, random_token_probability: float = 0.10,
                 keep_probability: float = 0.10, *, target_rows: Optional[int] = None,
                 batch_size: Optional[int] = None,
                 extra_excluded_token_ids: Optional[Iterable[int]] = None, seed: int | None = None):
        super().__init__(tokenizer, mlm_probability, mask_token_probability, random_token_probability,
                         keep_probability, extra_excluded_token_ids, seed)
        self.max_seq_len = int(max_seq_len)
        self.target_rows = target_rows
        self.dropped_sequences = 0
        if target_rows is not None:
            if batch_size is None:
                raise ValueError("batch_size must be provided when target_rows is set "
                                 "(needed to fix cu_seqlens length).")
            self.F = int(target_rows) * self.max_seq_len
            self.batch_size = int(batch_size)
            self.cu_len = self.batch_size + 1 + int(target_rows)

    def _pack_sequences(self, examples: Sequence[dict]):
        """Returns (input_ids (R,W), attention_mask (R,W), cu_seqlens, max_seqlen) — dynamic layout."""
        seqs = [_example_ids(e) for e in examples]
        W = self.max_seq_len
        lens = np.minimum(np.fromiter((len(s) for s in seqs), np.int32, len(seqs)), W)
        order, row_of, start_of, n_rows = pack_ffd(lens, W)
        ids = np.full((n_rows, W), self.pad_token_id, dtype=np.int64)
        att = np.zeros((n_rows, W), dtype=np.int64)
        for k in range(len(seqs)):
            s, r, c = int(order[k]), int(row_of[k]), int(start_of[k])
            n = int(lens[s])
            ids[r, c:c + n] = seqs[s][:n]
            att[r, c:c + n] = 1
        cu = np.zeros(len(seqs) + 1, dtype=np.int32)
        np.cumsum(lens[order], out=cu[1:])
        return (torch.from_numpy(ids), torch.from_numpy(att), torch.from_numpy(cu),
                int(lens.max()) if len(lens) else 0)

    def __call__(self, examples: Sequence[dict]) -> dict:
        W = self.max_seq_len
        if self.target_rows is None:
            ids, att, cu, max_seqlen = self._pack_sequences(examples)
            new_ids, labels = self.masker(ids.numpy(), self.rng(), forbid=att.numpy() == 0)
            return {"input_ids": torch.from_numpy(new_ids), "attention_mask": att,
                    "labels": torch.from_numpy(labels), "cu_seqlens": cu, "max_seqlen": max_seqlen}

        seqs = [_example_ids(e) for e in examples]
        lens = np.minimum(np.fromiter((len(s) for s in seqs), np.int32, len(seqs)), W)
        order, row_of, _, n_rows = pack_ffd(lens, W)
        n_keep = len(seqs)
        if n_rows > self.target_rows:
            n_keep = int(np.searchsorted(row_of, self.target_rows, side="left"))
            self.dropped_sequences += len(seqs) - n_keep
        flat, pos, cu = flatten(seqs, order, n_keep, W)
        T = len(flat)
        new_ids, labels = self.masker(flat, self.rng())
        F = self.F
        out_ids = np.full(F, self.pad_token_id, dtype=np.int64)
        out_lab = np.full(F, -100, dtype=np.int64)
        out_pos = np.zeros(F, dtype=np.int32)
        out_ids[:T], out_lab[:T], out_pos[:T] = new_ids, labels, pos
        cu_fixed = static_cu_seqlens(cu, F, W, self.cu_len)
        midx = np.nonzero(out_lab != -100)[0].astype(np.int32)
        return {"input_ids": torch.from_numpy(out_ids), "labels": torch.from_numpy(out_lab),
                "position_ids": torch.from_numpy(out_pos), "cu_seqlens": torch.from_numpy(cu_fixed),
                "max_seqlen": W, "masked_idx": torch.from_numpy(midx),
                "masked_labels": torch.from_numpy(out_lab[midx].astype(np.int32)),
                "num_real_tokens": T}
