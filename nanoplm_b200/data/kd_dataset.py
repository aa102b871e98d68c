"""Distillation datasets (reference: src/nanoplm/distillation/dataset.py).

* `KDDatasetOnTheFly`: iterates a FASTA file and yields raw sequences (teacher embeddings are
  computed during training); sharded over ranks and DataLoader workers.
* `SaveKDDataset`: FASTA -> stored teacher embeddings. Per sequence: `input_ids` (student tokens,
  int8), `attention_mask` (int8), `teacher_embeddings` (fp16, [max_seq_len, 1024]), all padded to
  max_seq_len. Container: HDF5 with one group per sequence ("0", "1", ...), the reference's layout,
  when h5py is installed; otherwise the same arrays in numpy `.kdz` archives (one per shard).
* `LoadKDDataset`: random access over a single file or `<stem>_shard_<k>` files, with an LRU pool of
  open shards and chunked prefetch.
* `shard_h5_file`: splits one big file into n shards.
"""
from __future__ import annotations

import bisect
import threading
from pathlib import Path
from typing import Iterator, Optional

import numpy as np
import torch
from torch.utils.data import Dataset, IterableDataset

from .fasta import iter_fasta
from .file_pool import ThreadSafeFileHandlePool
from .tokenizer import StudentTokenizer, TeacherTokenizer


def have_h5py() -> bool:
    try:
        import h5py  # noqa: F401
        return True
    except ImportError:
        return False


class _KdzFile:
    """Read-only view of a `.kdz` archive with the group-per-sequence interface of the HDF5 layout.

    An npz member is decompressed as a whole on every access and the underlying zip handle is not
    safe for concurrent readers (the prefetch thread and the main thread share one handle), so the
    three arrays are read once, under a lock, and served from memory afterwards."""

    _KEYS = ("input_ids", "attention_mask", "teacher_embeddings")

    def __init__(self, path):
        self._path = str(path)
        self._lock = threading.Lock()
        self._arrays: Optional[dict] = None
        with np.load(self._path, allow_pickle=False) as z:
            self.n = int(z["input_ids"].shape[0])

    def _load(self) -> dict:
        with self._lock:
            if self._arrays is None:
                with np.load(self._path, allow_pickle=False) as z:
                    self._arrays = {k: np.asarray(z[k]) for k in self._KEYS}
            return self._arrays

    def keys(self):
        return [str(i) for i in range(self.n)]

    def __len__(self):
        return self.n

    def __getitem__(self, key):
        i = int(key)
        arrays = self._load()
        return {k: arrays[k][i] for k in self._KEYS}

    def close(self):
        with self._lock:
            self._arrays = None


def open_kd_file(path):
    p = Path(path)
    if p.suffix == ".kdz":
        return _KdzFile(p)
    import h5py
    return h5py.File(p, "r")


def count_kd_sequences(path) -> int:
    f = open_kd_file(path)
    try:
        return len(f.keys())
    finally:
        f.close()


class KDDatasetOnTheFly(IterableDataset):
    def __init__(self, fasta_path, max_seqs_num: Optional[int] = None, rank: int = 0, world: int = 1):
        self.fasta_path = str(fasta_path)
        if not Path(self.fasta_path).exists():
            raise FileNotFoundError(f"FASTA file not found: {self.fasta_path}")
        self.max_seqs_num, self.rank, self.world = max_seqs_num, rank, world

    def __iter__(self) -> Iterator[dict]:
        info = torch.utils.data.get_worker_info()
        nw, wid = (info.num_workers, info.id) if info else (1, 0)
        stride, offset = self.world * nw, self.rank * nw + wid
        for i, (_, seq) in enumerate(iter_fasta(self.fasta_path)):
            if self.max_seqs_num is not None and i >= self.max_seqs_num:
                break
            if i % stride == offset:
                yield {"raw_sequence": seq}


class SaveKDDataset:
    def __init__(self, input_fasta, output_path, max_seq_len: int = 512, batch_size: int = 4,
                 device: str = "auto", samples_per_shard: int = -1, teacher=None,
                 random_init_teacher: bool = False, force: bool = False, skip_n: int = 0):
        self.input_fasta, self.output_path = Path(input_fasta), Path(output_path)
        self.skip_n = max(0, int(skip_n))
        if not self.input_fasta.exists():
            raise FileNotFoundError(f"FASTA file not found: {self.input_fasta}")
        self.max_seq_len, self.batch_size = int(max_seq_len), int(batch_size)
        self.samples_per_shard, self.force = int(samples_per_shard), force
        if device == "auto":
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self._teacher, self._random_init = teacher, random_init_teacher
        self.student_tok, self.teacher_tok = StudentTokenizer(), TeacherTokenizer()
        self.use_h5 = have_h5py() and self.output_path.suffix != ".kdz"

    def _get_teacher(self):
        if self._teacher is None:
            from nanoplm_b200.models.teacher import T5EncoderTeacher
            if self._random_init:
                self._teacher = T5EncoderTeacher(random_init=True)
            else:
                self._teacher = T5EncoderTeacher.from_pretrained("Rostlab/prot_t5_xl_uniref50")
            self._teacher.to(self.device)
            if self.device.type == "cuda":
                self._teacher.to(torch.bfloat16)
        elif hasattr(self._teacher, "encoder_model"):
            self._teacher = self._teacher.encoder_model      # a `ProtT5`-style wrapper
        return self._teacher

    def _shard_path(self, k: Optional[int]) -> Path:
        suffix = ".h5" if self.use_h5 else ".kdz"
        stem = self.output_path.with_suffix("")
        return Path(f"{stem}{suffix}") if k is None else Path(f"{stem}_shard_{k:04d}{suffix}")

    def _write(self, path: Path, ids, mask, emb) -> None:
        path.parent.mkdir(parents=True, exist_ok=True)
        if self.use_h5:
            import h5py
            with h5py.File(path, "w") as h:
                for i in range(len(ids)):
                    g = h.create_group(str(i))
                    g.create_dataset("input_ids", data=ids[i])
                    g.create_dataset("attention_mask", data=mask[i])
                    g.create_dataset("teacher_embeddings", data=emb[i])
        else:
            with open(path, "wb") as f:
                np.savez(f, input_ids=np.stack(ids), attention_mask=np.stack(mask), teacher_embeddings=np.stack(emb))

    @torch.no_grad()
    def run(self) -> list[Path]:
        existing = list(self.output_path.parent.glob(self.output_path.stem + "*"))
        if existing and not self.force:
            raise FileExistsError(f"Output already exists: {existing[0]}. Use --force to overwrite.")
        for f in existing:
            f.unlink()
        teacher = self._get_teacher()
        L = self.max_seq_len
        seqs = [s for _, s in iter_fasta(self.input_fasta)][self.skip_n:]
        files, ids_buf, mask_buf, emb_buf, shard = [], [], [], [], 0

        def flush(final: bool):
            nonlocal shard, ids_buf, mask_buf, emb_buf
            if not ids_buf:
                return
            single = self.samples_per_shard <= 0
            path = self._shard_path(None if single else shard)
            self._write(path, ids_buf, mask_buf, emb_buf)
            files.append(path)
            shard += 1
            ids_buf, mask_buf, emb_buf = [], [], []

        for i in range(0, len(seqs), self.batch_size):
            batch = seqs[i:i + self.batch_size]
            st = self.student_tok(batch, padding="max_length", max_length=L, truncation=True, return_tensors="pt")
            tt = self.teacher_tok([teacher.preprocess(s) for s in batch], padding="max_length", max_length=L,
                                  truncation=True, return_tensors="pt")
            emb = teacher(tt["input_ids"].to(self.device), tt["attention_mask"].to(self.device))
            emb = emb.float().cpu().numpy().astype(np.float16)
            for b in range(len(batch)):
                ids_buf.append(st["input_ids"][b].numpy().astype(np.int8))
                mask_buf.append(st["attention_mask"][b].numpy().astype(np.int8))
                emb_buf.append(emb[b])
                if self.samples_per_shard > 0 and len(ids_buf) >= self.samples_per_shard:
                    flush(False)
        flush(True)
        return files


class LoadKDDataset(Dataset):
    def __init__(self, path_or_prefix, max_open_files: int = 5, chunk_size: int = 32, prefetch_batches: int = 2,
                 use_threading: bool = True, seed: Optional[int] = None, sharded: Optional[bool] = None):
        p = Path(path_or_prefix)
        stem = p.with_suffix("")
        shards = sorted(p.parent.glob(f"{stem.name}_shard_*.h5")) + sorted(p.parent.glob(f"{stem.name}_shard_*.kdz"))
        singles = [q for q in (Path(f"{stem}.h5"), Path(f"{stem}.kdz")) if q.exists()]
        self.files = [str(f) for f in (shards if shards and sharded is not False else singles or shards)]
        if not self.files:
            raise FileNotFoundError(f"No KD dataset files found for {path_or_prefix}")
        self.pool = ThreadSafeFileHandlePool(max_open_files, opener=open_kd_file)
        self.counts = [count_kd_sequences(f) for f in self.files]
        self.cum = np.cumsum(self.counts)
        self.chunk_size, self.prefetch_batches, self.use_threading = chunk_size, prefetch_batches, use_threading
        self._order = np.arange(int(self.cum[-1]))
        if seed is not None:
            np.random.default_rng(seed).shuffle(self._order)
        self._cache: dict[int, dict] = {}
        self._cache_lock = threading.Lock()

    def __len__(self) -> int:
        return int(self.cum[-1])

    def _locate(self, gi: int) -> tuple[int, int]:
        s = bisect.bisect_right(self.cum, gi)
        return s, gi - (int(self.cum[s - 1]) if s else 0)

    def _read(self, gi: int) -> dict:
        s, l = self._locate(gi)
        g = self.pool.get(self.files[s])[str(l)]
        return {"input_ids": torch.from_numpy(np.asarray(g["input_ids"]).astype(np.int64)),
                "attention_mask": torch.from_numpy(np.asarray(g["attention_mask"]).astype(np.int64)),
                "teacher_embeddings": torch.from_numpy(np.asarray(g["teacher_embeddings"]).astype(np.float32))}

    def _prefetch(self, start: int) -> None:
        end = min(len(self), start + self.chunk_size * max(1, self.prefetch_batches))
        for i in range(start, end):
            gi = int(self._order[i])
            with self._cache_lock:
                if gi in self._cache:
                    continue
            item = self._read(gi)
            with self._cache_lock:
                if len(self._cache) > 8 * self.chunk_size:
                    self._cache.pop(next(iter(self._cache)))
                self._cache[gi] = item

    def __getitem__(self, idx: int) -> dict:
        if idx < 0 or idx >= len(self):
            raise IndexError(idx)
        gi = int(self._order[idx])
        with self._cache_lock:
            item = self._cache.pop(gi, None)
        if item is None:
            item = self._read(gi)
        if self.use_threading and idx % self.chunk_size == 0:
            threading.Thread(target=self._prefetch, args=(idx + 1,), daemon=True).start()
        return item

    def stats(self) -> dict:
        return {"files": len(self.files), "sequences": len(self), **self.pool.stats()}

    def __getstate__(self):
        d = self.__dict__.copy()
        d["_cache"], d["_cache_lock"] = {}, None
        return d

    def __setstate__(self, d):
        self.__dict__.update(d)
        self._cache_lock = threading.Lock()


def shard_h5_file(input_path, n_shards: int, output_dir=None, total: Optional[int] = None) -> list[Path]:
    src_path = Path(input_path)
    if not src_path.exists():
        raise FileNotFoundError(f"Input file not found: {src_path}")
    if n_shards < 1:
        raise ValueError("n_shards must be >= 1")
    out_dir = Path(output_dir) if output_dir else src_path.parent
    out_dir.mkdir(parents=True, exist_ok=True)
    src = open_kd_file(src_path)
    keys = sorted(src.keys(), key=int)
    total = total or len(keys)
    per = -(-total // n_shards)
    files = []
    use_h5 = src_path.suffix != ".kdz" and have_h5py()
    for k in range(n_shards):
        part = keys[k * per:(k + 1) * per]
        if not part:
            break
        dst = out_dir / f"{src_path.stem}_shard_{k:04d}{src_path.suffix}"
        if use_h5:
            import h5py
            with h5py.File(dst, "w") as h:
                for j, key in enumerate(part):
                    src.copy(src[key], h, name=str(j))
        else:
            rows = [src[key] for key in part]
            with open(dst, "wb") as f:
                np.savez(f, **{name: np.stack([np.asarray(r[name]) for r in rows])
                               for name in ("input_ids", "attention_mask", "teacher_embeddings")})
        files.append(dst)
    src.close()
    return files
