"""Minimal FASTA reader / writer / random-access index in pure Python (no Biopython).

`iter_fasta` streams (header, sequence) records; `FastaIndex` records the byte offset of every
record so that a record can be fetched without scanning, which is what sharded tokenisation and
shuffling need (the reference uses Biopython's SQLite index for the same purpose,
src/nanoplm/pretraining/dataset.py:70-72, src/nanoplm/data/shuffler.py:97-124).
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator

import numpy as np


def iter_fasta(path: str | Path) -> Iterator[tuple[str, str]]:
    header, chunks = None, []
    with open(path, "r", encoding="utf-8", errors="replace") as f:
        for line in f:
            line = line.rstrip("\r\n")
            if not line:
                continue
            if line[0] == ">":
                if header is not None:
                    yield header, "".join(chunks)
                header, chunks = line[1:], []
            elif header is not None:
                chunks.append(line.strip())
    if header is not None:
        yield header, "".join(chunks)


def count_fasta(path: str | Path) -> int:
    n = 0
    with open(path, "rb") as f:
        for line in f:
            if line[:1] == b">":
                n += 1
    return n


def write_fasta(records, path: str | Path, width: int = 60) -> int:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    n = 0
    with open(p, "w", encoding="utf-8") as f:
        for header, seq in records:
            f.write(f">{header}\n")
            if width and width > 0:
                for i in range(0, len(seq), width):
                    f.write(seq[i:i + width] + "\n")
            else:
                f.write(seq + "\n")
            n += 1
    return n


class FastaIndex:
    """Byte offsets of all records of a FASTA file; `get(i)` reads one record."""

    def __init__(self, path: str | Path):
        self.path = str(path)
        starts = []
        pos = 0
        with open(self.path, "rb") as f:
            for line in f:
                if line[:1] == b">":
                    starts.append(pos)
                pos += len(line)
        self.size = pos
        self.starts = np.asarray(starts, dtype=np.int64)

    def __len__(self) -> int:
        return len(self.starts)

    def raw(self, i: int) -> bytes:
        a = int(self.starts[i])
        b = int(self.starts[i + 1]) if i + 1 < len(self.starts) else self.size
        with open(self.path, "rb") as f:
            f.seek(a)
            return f.read(b - a)

    def get(self, i: int) -> tuple[str, str]:
        lines = self.raw(i).decode("utf-8", errors="replace").splitlines()
        return lines[0][1:], "".join(s.strip() for s in lines[1:])
