"""Seeded synthetic protein data for benchmarks and tests (no network, no real dataset needed).

Residues are drawn i.i.d. from the 20 canonical amino acids at their natural composition
frequencies (UniProtKB/Swiss-Prot statistics: L 9.9 %, A 8.3 %, G 7.1 %, ... W 1.3 %); lengths are
uniform in [min_len, max_len]. `write_synthetic_fasta` and `write_synthetic_dataset` produce files in
the same formats the data-preparation CLI writes, so the training pipelines run on them unchanged.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

from .manifest import PretrainManifest, write_manifest
from .tokenizer import ProtTokenizer

AA_FREQ = {
    "L": 9.87, "A": 8.25, "G": 7.07, "V": 6.86, "E": 6.72, "S": 6.65, "I": 5.91, "K": 5.80,
    "R": 5.53, "D": 5.46, "T": 5.36, "P": 4.74, "N": 4.06, "Q": 3.93, "F": 3.86, "Y": 2.92,
    "M": 2.41, "H": 2.27, "C": 1.38, "W": 1.10,
}
_LETTERS = np.frombuffer("".join(AA_FREQ).encode(), dtype=np.uint8)
_PROBS = np.asarray(list(AA_FREQ.values()), dtype=np.float64)
_PROBS /= _PROBS.sum()


def synthetic_sequences(n: int, min_len: int = 20, max_len: int = 512, seed: int = 0) -> list[str]:
    rng = np.random.default_rng(seed)
    lens = rng.integers(min_len, max_len + 1, size=n)
    return [_LETTERS[rng.choice(len(_LETTERS), size=int(l), p=_PROBS)].tobytes().decode() for l in lens]


def synthetic_token_sequences(n: int, min_len: int = 20, max_len: int = 512, seed: int = 0,
                              use_bos: bool = False) -> list[np.ndarray]:
    """Token ids (uint8) including the trailing </s> (and leading <s> when use_bos)."""
    tok = ProtTokenizer(use_bos_token=use_bos)
    return [tok.encode_np(s) for s in synthetic_sequences(n, min_len, max_len, seed)]


def write_synthetic_fasta(path, n: int, min_len: int = 20, max_len: int = 512, seed: int = 0) -> Path:
    from .fasta import write_fasta
    seqs = synthetic_sequences(n, min_len, max_len, seed)
    write_fasta(((f"syn{i}", s) for i, s in enumerate(seqs)), path)
    return Path(path)


def write_synthetic_dataset(out_dir, n_train: int, n_val: int, min_len: int = 20, max_len: int = 512,
                            seed: int = 0, samples_per_shard: int = 10000, use_bos: bool = False) -> Path:
    """Writes train/ and val/ shard directories plus the .data_manifest (max_seq_len counts the
    special tokens, like the tokenizer's max_length)."""
    out = Path(out_dir)
    extra = 2 if use_bos else 1
    for split, n, s in (("train", n_train, seed), ("val", n_val, seed + 1)):
        d = out / split
        d.mkdir(parents=True, exist_ok=True)
        seqs = synthetic_token_sequences(n, min_len, max_len, s, use_bos)
        for k in range(0, len(seqs), samples_per_shard):
            part = seqs[k:k + samples_per_shard]
            i = k // samples_per_shard
            np.concatenate(part).astype(np.uint8).tofile(d / f"shard_{i:04d}.bin")
            np.save(d / f"shard_{i:04d}.idx.npy", np.asarray([len(p) for p in part], dtype=np.int32))
    write_manifest(out, PretrainManifest(
        pipeline_mode="pretrain", seqs_num=n_train + n_val, min_seq_len=min_len,
        max_seq_len=max_len + extra, val_ratio=n_val / max(1, n_train + n_val), train_dir="train",
        val_dir="val", train_sequences=n_train, val_sequences=n_val, sharded=True,
        samples_per_shard=samples_per_shard))
    return out
