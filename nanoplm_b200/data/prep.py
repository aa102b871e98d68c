"""FASTA preparation steps behind `nanoplm data download|extract|shuffle|filter|split`.

Behavioural parity with the reference's step classes (src/nanoplm/data/downloader.py,
extractor.py, shuffler.py, filterer.py, splitor.py): same inputs, outputs and error cases; the
in-process shuffle is seeded (the reference stores the seed but never applies it,
data/shuffler.py:40,109).
"""
from __future__ import annotations

import gzip
import random
import shutil
import ssl
import subprocess
import urllib.request
from pathlib import Path
from typing import Optional

from .fasta import FastaIndex, iter_fasta, write_fasta


class DownloadError(RuntimeError):
    pass


class ExtractionError(RuntimeError):
    pass


class ShufflingError(RuntimeError):
    pass


class FilterError(RuntimeError):
    pass


class SplitError(RuntimeError):
    pass


class Downloader:
    def __init__(self, url: str, output_path: str | Path, chunk_size: int = 1 << 16):
        self.url, self.output_path, self.chunk_size = url, Path(output_path), chunk_size

    def download(self, progress=None) -> Path:
        self.output_path.parent.mkdir(parents=True, exist_ok=True)
        try:
            try:
                import certifi
                ctx = ssl.create_default_context(cafile=certifi.where())
            except Exception:
                ctx = ssl.create_default_context()
            tmp = self.output_path.with_suffix(self.output_path.suffix + ".part")
            with urllib.request.urlopen(self.url, context=ctx) as resp, open(tmp, "wb") as out:
                while True:
                    chunk = resp.read(self.chunk_size)
                    if not chunk:
                        break
                    out.write(chunk)
                    if progress is not None:
                        progress(len(chunk))
            tmp.replace(self.output_path)
        except Exception as exc:
            raise DownloadError(f"Failed to download {self.url}: {exc}") from exc
        return self.output_path


class Extractor:
    def __init__(self, input_path: str | Path, output_path: str | Path):
        self.input_path, self.output_path = Path(input_path), Path(output_path)

    def extract(self) -> Path:
        if not self.input_path.exists():
            raise ExtractionError(f"Input file not found: {self.input_path}")
        self.output_path.parent.mkdir(parents=True, exist_ok=True)
        try:
            with gzip.open(self.input_path, "rb") as src, open(self.output_path, "wb") as dst:
                shutil.copyfileobj(src, dst, 1 << 20)
        except (OSError, EOFError) as exc:
            raise ExtractionError(f"Failed to extract {self.input_path}: {exc}") from exc
        return self.output_path


class FastaShuffler:
    """Shuffles the records of a FASTA file. backend "biopython" is the in-process path (kept under
    that name for CLI compatibility); "seqkit" shells out to the external binary."""

    def __init__(self, input_path, output_path, backend: str = "biopython", seed: Optional[int] = 24,
                 threads: int = 4):
        self.input_path, self.output_path = Path(input_path), Path(output_path)
        # no seed: one is drawn and kept, as the reference does (data/shuffler.py:40)
        self.seed = int(seed) if seed else random.randint(1, 1000)
        self.backend, self.threads = backend, threads

    def shuffle(self) -> Path:
        if not self.input_path.exists():
            raise ShufflingError(f"Input FASTA not found: {self.input_path}")
        self.output_path.parent.mkdir(parents=True, exist_ok=True)
        if self.backend == "seqkit":
            exe = shutil.which("seqkit")
            if exe is None:
                raise ShufflingError("seqkit backend requested but the seqkit binary is not on PATH")
            cmd = [exe, "shuffle", "--threads", str(self.threads), "--two-pass", "--rand-seed",
                   str(self.seed), "-o", str(self.output_path), str(self.input_path)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise ShufflingError(f"seqkit failed: {proc.stderr.strip()}")
            return self.output_path
        if self.backend not in ("biopython", "python"):
            raise ShufflingError(f"Unknown shuffle backend: {self.backend}")
        index = FastaIndex(self.input_path)
        order = list(range(len(index)))
        random.Random(self.seed).shuffle(order)
        with open(self.output_path, "wb") as out:
            for i in order:
                rec = index.raw(i)
                out.write(rec if rec.endswith(b"\n") else rec + b"\n")
        return self.output_path


class Filterer:
    def __init__(self, input_path, output_path, min_seq_len: int = 20, max_seq_len: int = 512,
                 seqs_num: int = -1, skip_n: int = 0):
        self.input_path, self.output_path = Path(input_path), Path(output_path)
        self.min_seq_len, self.max_seq_len = int(min_seq_len), int(max_seq_len)
        self.seqs_num, self.skip_n = int(seqs_num), int(skip_n)
        if self.min_seq_len > self.max_seq_len:
            raise FilterError("min_seq_len must be <= max_seq_len")

    def filter(self) -> dict:
        if not self.input_path.exists():
            raise FilterError(f"Input FASTA not found: {self.input_path}")
        seen = kept = 0

        def gen():
            nonlocal seen, kept
            for i, (h, s) in enumerate(iter_fasta(self.input_path)):
                if i < self.skip_n:
                    continue
                seen += 1
                if self.min_seq_len <= len(s) <= self.max_seq_len:
                    kept += 1
                    yield h, s
                    if self.seqs_num != -1 and kept >= self.seqs_num:
                        return
        write_fasta(gen(), self.output_path)
        return {"processed": seen, "kept": kept}


class Splitor:
    def __init__(self, input_path, output_dir, val_ratio: float = 0.1):
        self.input_path, self.output_dir, self.val_ratio = Path(input_path), Path(output_dir), float(val_ratio)
        if not 0.0 <= self.val_ratio < 1.0:
            raise SplitError("val_ratio must be in [0, 1)")

    def split(self) -> tuple[int, int]:
        if not self.input_path.exists():
            raise SplitError(f"Input FASTA not found: {self.input_path}")
        recs = list(iter_fasta(self.input_path))
        n_val = int(len(recs) * self.val_ratio)
        n_train = len(recs) - n_val
        write_fasta(recs[:n_train], self.output_dir / "train.fasta")
        write_fasta(recs[n_train:], self.output_dir / "val.fasta")
        return n_train, n_val
