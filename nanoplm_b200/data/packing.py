"""Sequence packing for varlen attention.

`pack_ffd` is first-fit-decreasing bin packing into rows of `width` tokens (C++,
nanoplm_b200/csrc/packer.cpp). `pack_static` assembles the flat, fixed-size batch the model
consumes: `input_ids (F,)`, `position_ids (F,)`, fixed-length `cu_seqlens` where the padding tail
is carved into pseudo-sequences of at most `width` tokens. Formats follow the reference collator
(src/nanoplm/pretraining/collator.py:250-327, 405-458); unlike it, a batch whose real tokens exceed
F = target_rows * width is handled (whole rows beyond target_rows are dropped and counted) rather
than failing on a shape mismatch.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import numpy as np

from nanoplm_b200.ops._lib import lib

_I32P = ctypes.POINTER(ctypes.c_int32)
_I64P = ctypes.POINTER(ctypes.c_int64)
_U8P = ctypes.POINTER(ctypes.c_uint8)


def pack_ffd(lengths: np.ndarray, width: int):
    """Returns (order, row_of, start_of, n_rows) — see packer.cpp."""
    lens = np.ascontiguousarray(lengths, dtype=np.int32)
    n = len(lens)
    order = np.empty(n, dtype=np.int32)
    row_of = np.empty(n, dtype=np.int32)
    start_of = np.empty(n, dtype=np.int32)
    n_rows = lib("packer").nplm_pack_ffd(
        lens.ctypes.data_as(_I32P), ctypes.c_int(n), ctypes.c_int(int(width)),
        order.ctypes.data_as(_I32P), row_of.ctypes.data_as(_I32P), start_of.ctypes.data_as(_I32P))
    return order, row_of, start_of, int(n_rows)


def pack_ffd_python(lengths: Sequence[int], width: int):
    """Reference implementation in plain Python (test oracle for the C++ packer)."""
    idx = sorted(range(len(lengths)), key=lambda i: lengths[i], reverse=True)
    rows: list[list[int]] = []
    fill: list[int] = []
    for i in idx:
        n = min(int(lengths[i]), width)
        for r in range(len(rows)):
            if fill[r] + n <= width:
                rows[r].append(i)
                fill[r] += n
                break
        else:
            rows.append([i])
            fill.append(n)
    order = [i for row in rows for i in row]
    row_of = [r for r, row in enumerate(rows) for _ in row]
    return order, row_of, len(rows)


# cost(len) = len + len^2 / 2700: measured on the default encoder (one B200), a token costs about
# 1.23 us in the token-wise kernels and a (query, key) pair of the six full-attention layers 0.45 ns
DEFAULT_QUADRATIC_COST = 1.0 / 2700.0


def balance_bins(lengths: np.ndarray, n_bins: int, per_bin: int, quad: float = DEFAULT_QUADRATIC_COST):
    """Deals len(lengths) == n_bins * per_bin sequences into bins of exactly per_bin sequences with
    (greedily) equal cost len + quad * len^2. Returns (bin_of int32[n], bin_cost float64[n_bins]).
    Deterministic: the same lengths give the same assignment on every rank."""
    lens = np.ascontiguousarray(lengths, dtype=np.int32)
    n = len(lens)
    bin_of = np.empty(n, dtype=np.int32)
    bin_cost = np.empty(n_bins, dtype=np.float64)
    rc = lib("packer").nplm_balance_bins(
        lens.ctypes.data_as(_I32P), ctypes.c_int(n), ctypes.c_int(int(n_bins)), ctypes.c_int(int(per_bin)),
        ctypes.c_double(float(quad)), bin_of.ctypes.data_as(_I32P),
        bin_cost.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
    if rc != 0:
        raise ValueError(f"balance_bins: {n} sequences do not fill {n_bins} bins of {per_bin}")
    return bin_of, bin_cost


def balance_bins_python(lengths: Sequence[int], n_bins: int, per_bin: int, quad: float = DEFAULT_QUADRATIC_COST):
    """Plain-Python restatement of balance_bins (test oracle)."""
    cost = [l + quad * float(l) * l for l in lengths]
    order = sorted(range(len(lengths)), key=lambda i: -cost[i])
    fill, total = [0] * n_bins, [0.0] * n_bins
    bin_of = [0] * len(lengths)
    for i in order:
        best = min((b for b in range(n_bins) if fill[b] < per_bin), key=lambda b: (total[b], b))
        bin_of[i] = best
        total[best] += cost[i]
        fill[best] += 1
    return bin_of, total


def flatten(seqs: Sequence[np.ndarray], order: np.ndarray, n_keep: int, width: int):
    """Concatenates sequences in `order[:n_keep]`; returns (flat_ids int64, pos int32, cu int32)."""
    lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=len(seqs))
    offsets = np.zeros(len(seqs) + 1, dtype=np.int64)
    np.cumsum(lens, out=offsets[1:])
    tokens = np.concatenate([np.asarray(s, dtype=np.uint8) for s in seqs]) if len(seqs) else np.zeros(0, np.uint8)
    total = int(np.minimum(lens[order[:n_keep]], width).sum()) if n_keep else 0
    flat = np.empty(total, dtype=np.int64)
    pos = np.empty(total, dtype=np.int32)
    cu = np.empty(n_keep + 1, dtype=np.int32)
    order = np.ascontiguousarray(order, dtype=np.int32)
    fn = lib("packer").nplm_pack_flatten
    fn.restype = ctypes.c_int64
    t = fn(
        tokens.ctypes.data_as(_U8P), offsets.ctypes.data_as(_I64P), order.ctypes.data_as(_I32P),
        ctypes.c_int(n_keep), ctypes.c_int(int(width)), flat.ctypes.data_as(_I64P),
        pos.ctypes.data_as(_I32P), cu.ctypes.data_as(_I32P))
    assert int(t) == total
    return flat, pos, cu


def static_cu_seqlens(cu_real: np.ndarray, flat_len: int, width: int, cu_len: int) -> np.ndarray:
    """Fixed-length cu_seqlens: real boundaries, then the padding tail split into chunks of at most
    `width`, then `flat_len` repeated (zero-length sequences)."""
    out = np.full(cu_len, flat_len, dtype=np.int32)
    n_real = min(len(cu_real), cu_len)
    out[:n_real] = cu_real[:n_real]
    pos = int(cu_real[-1])
    i = n_real
    while pos < flat_len and i < cu_len:
        pos = min(flat_len, pos + width)
        out[i] = pos
        i += 1
    return out
