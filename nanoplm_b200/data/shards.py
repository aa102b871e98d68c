"""Pre-tokenised binary shards: `shard_NNNN.bin` (uint8 token ids of all sequences back to back)
plus `shard_NNNN.idx.npy` (int32 length of every sequence).

On-disk format and class surface follow the reference (src/nanoplm/pretraining/dataset.py:17-322).
Tokenisation here is a numpy look-up table, so one process handles ~10^6 residues per millisecond
and no SQLite side index is written next to the FASTA file.
"""
from __future__ import annotations

import bisect
import os
from concurrent.futures import ProcessPoolExecutor
from math import ceil
from pathlib import Path

import numpy as np
import torch

from .fasta import FastaIndex
from .tokenizer import ProtTokenizer


def _write_shard(args) -> str:
    shard_idx, fasta_path, starts, size, first, last, use_bos, max_length, out_dir = args
    tok = ProtTokenizer(use_bos_token=use_bos)
    index = FastaIndex.__new__(FastaIndex)
    index.path, index.starts, index.size = fasta_path, starts, size
    chunks, lens = [], []
    for i in range(first, last):
        _, seq = index.get(i)
        ids = tok.encode_np(seq, add_special_tokens=True, max_length=max_length, truncation=True)
        chunks.append(ids)
        lens.append(len(ids))
    out = Path(out_dir)
    bin_path = out / f"shard_{shard_idx:04d}.bin"
    np.concatenate(chunks).astype(np.uint8).tofile(bin_path)
    np.save(out / f"shard_{shard_idx:04d}.idx.npy", np.asarray(lens, dtype=np.int32))
    return str(bin_path)


class ShardWriter:
    """FASTA -> binary shards. Not a Dataset: a one-off preprocessing step."""

    def __init__(self, fasta_path, tokenizer: ProtTokenizer, max_length: int, output_dir,
                 samples_per_shard: int = 10000, max_workers: int = -1, force: bool = False):
        self.fasta_path = str(fasta_path)
        self.tokenizer = tokenizer
        self.max_length = int(max_length)
        self.output_dir = Path(output_dir)
        self.samples_per_shard = int(samples_per_shard)
        self.max_workers = (os.cpu_count() or 1) if max_workers in (-1, None) else max(1, int(max_workers))
        self.force = bool(force)
        p = Path(self.fasta_path)
        if not p.exists():
            raise FileNotFoundError(f"FASTA file not found: {self.fasta_path}")
        if not p.is_file():
            raise ValueError(f"Path is not a file: {self.fasta_path}")
        if p.stat().st_size == 0:
            raise ValueError(f"FASTA file is empty: {self.fasta_path}")
        self._index = FastaIndex(self.fasta_path)
        if len(self._index) == 0:
            raise ValueError(f"No sequences found in FASTA: {self.fasta_path}")

    def __len__(self) -> int:
        return len(self._index)

    def create_shards(self) -> list[Path]:
        existing = self.output_dir.exists() and any(self.output_dir.glob("*.bin"))
        if existing and not self.force:
            raise FileExistsError(
                f"Binary shards already exist in {self.output_dir}. Set force=True to overwrite them.")
        if existing:
            for f in list(self.output_dir.glob("*.bin")) + list(self.output_dir.glob("*.idx.npy")):
                f.unlink()
        self.output_dir.mkdir(parents=True, exist_ok=True)
        total = len(self._index)
        n_shards = ceil(total / self.samples_per_shard)
        use_bos = bool(getattr(self.tokenizer, "use_bos_token", False))
        jobs = [(i, self.fasta_path, self._index.starts, self._index.size,
                 i * self.samples_per_shard, min(total, (i + 1) * self.samples_per_shard), use_bos,
                 self.max_length, str(self.output_dir)) for i in range(n_shards)]
        if self.max_workers == 1 or n_shards == 1:
            paths = [_write_shard(j) for j in jobs]
        else:
            with ProcessPoolExecutor(max_workers=min(self.max_workers, n_shards)) as ex:
                paths = list(ex.map(_write_shard, jobs))
        return [Path(p) for p in paths]


class LazyFastaDataset(torch.utils.data.Dataset):
    """Tokenises the records of a FASTA file on access, without a sharding step: small datasets,
    quick experiments, and the oracle the shards are compared with. Same examples as `ShardedDataset`
    (`input_ids` / `attention_mask` of one sequence, truncated to `max_length`). The class left the
    reference's package while its tests still describe it (tests/test_fasta_dataset.py:16-103,
    236-265): three-argument constructor, `max_length` attribute, IndexError for negative and
    out-of-range indices, ValueError for an empty file. Pickles to its arguments, so DataLoader
    workers index the file themselves."""

    def __init__(self, fasta_path, tokenizer: ProtTokenizer, max_length: int):
        self.fasta_path, self.tokenizer, self.max_length = str(fasta_path), tokenizer, int(max_length)
        p = Path(self.fasta_path)
        if not p.exists():
            raise FileNotFoundError(f"FASTA file not found: {self.fasta_path}")
        if p.stat().st_size == 0:
            raise ValueError(f"FASTA file is empty: {self.fasta_path}")
        self._index = FastaIndex(self.fasta_path)
        if len(self._index) == 0:
            raise ValueError(f"FASTA file is empty: {self.fasta_path} holds no records")

    def __getstate__(self):
        return (self.fasta_path, self.tokenizer, self.max_length)

    def __setstate__(self, state):
        self.__init__(*state)

    def __len__(self) -> int:
        return len(self._index)

    def __getitem__(self, idx: int) -> dict:
        if idx < 0 or idx >= len(self):
            raise IndexError(f"Index {idx} out of bounds for dataset of size {len(self)}")
        _, seq = self._index.get(int(idx))
        enc = self.tokenizer(seq, add_special_tokens=True, truncation=True, max_length=self.max_length)
        ids = torch.as_tensor(enc["input_ids"], dtype=torch.long)
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids)}


class ShardedDataset(torch.utils.data.Dataset):
    """Memory-mapped view over a directory of shards. Pickles to just the directory path so that
    DataLoader workers re-open the maps themselves."""

    def __init__(self, data_dir):
        self._open(str(data_dir))

    def _open(self, data_dir: str) -> None:
        self.data_dir = Path(data_dir)
        if not self.data_dir.exists():
            raise FileNotFoundError(f"Data directory not found: {self.data_dir}")
        if not self.data_dir.is_dir():
            raise ValueError(f"Path is not a directory: {self.data_dir}")
        self._bin_paths = [str(p) for p in sorted(self.data_dir.glob("*.bin"))]
        if not self._bin_paths:
            raise FileNotFoundError(f"No binary shard files (*.bin) found in {self.data_dir}")
        self._offsets, self.lengths = [], []
        for bp in self._bin_paths:
            ip = Path(bp).with_name(Path(bp).stem + ".idx.npy")
            if not ip.exists():
                raise FileNotFoundError(f"Index file not found for shard: {ip}")
            sizes = np.load(str(ip)).astype(np.int64)
            self._offsets.append(np.concatenate([[0], np.cumsum(sizes)]))
            self.lengths.append(len(sizes))
        self.cum_lengths = np.cumsum(self.lengths)
        self._mmaps = None

    def __getstate__(self):
        return str(self.data_dir)

    def __setstate__(self, state):
        self._open(state)

    def __len__(self) -> int:
        return int(self.cum_lengths[-1])

    def sequence_lengths(self) -> np.ndarray:
        """Token count of every sequence, in dataset order (used by length-aware batching)."""
        return np.concatenate([np.diff(o) for o in self._offsets]).astype(np.int32)

    def _locate(self, idx: int) -> tuple[int, int]:
        s = bisect.bisect_right(self.cum_lengths, idx)
        return s, idx - (int(self.cum_lengths[s - 1]) if s > 0 else 0)

    def get_np(self, idx: int) -> np.ndarray:
        if idx < 0 or idx >= len(self):
            raise IndexError(f"Index {idx} out of bounds for dataset of size {len(self)}")
        if self._mmaps is None:
            self._mmaps = [np.memmap(p, dtype=np.uint8, mode="r") for p in self._bin_paths]
        s, l = self._locate(idx)
        off = self._offsets[s]
        return np.array(self._mmaps[s][int(off[l]):int(off[l + 1])])

    def __getitem__(self, idx: int) -> dict:
        ids = torch.from_numpy(self.get_np(idx))
        return {"input_ids": ids, "attention_mask": (ids != 0).to(torch.uint8)}
