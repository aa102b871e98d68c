"""Pre-flight validation of prepared datasets (reference: src/nanoplm/data/validation.py).

Pretraining shards: every `.bin` has an `.idx.npy`, the index is a non-empty 1-D array, and the
lengths sum to the size of the `.bin` file. Distillation datasets: the FASTA files (on-the-fly) or
the HDF5 shards (pre-computed) named by the manifest exist.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

from .manifest import (DistillationManifest, PretrainManifest, read_manifest,
                       validate_manifest_for_pipeline)


class ValidationError(Exception):
    pass


class ShardInfo(dict):
    """Result of `validate_pretrain_shards`: counts by key (`num_shards`, `num_sequences`) and, like
    the reference's return value (data/validation.py:182-295), the sorted `.bin` paths when iterated
    or measured with `len()` / indexed by position."""

    def __init__(self, bins: list[Path], num_sequences: int):
        super().__init__(num_shards=len(bins), num_sequences=num_sequences)
        self.paths = list(bins)

    def __iter__(self):
        return iter(self.paths)

    def __len__(self):
        return len(self.paths)

    def __getitem__(self, k):
        return self.paths[k] if isinstance(k, (int, slice)) else dict.__getitem__(self, k)


def validate_pretrain_shards(shard_dir: str | Path, expected_count: int | None = None,
                             check_contents: bool = True, label: str = "shards") -> ShardInfo:
    d = Path(shard_dir)
    if not d.exists():
        raise ValidationError(f"{label} directory not found: {d}")
    if not d.is_dir():
        raise ValidationError(f"{label} path is not a directory: {d}")
    bins = sorted(d.glob("*.bin"))
    if not bins:
        raise ValidationError(f"No binary shard files (*.bin) found in {d}")
    if expected_count is not None and len(bins) != expected_count:
        raise ValidationError(f"Expected {expected_count} shard files in {d}, found {len(bins)}")
    total = 0
    for b in bins:
        idx = b.with_name(b.stem + ".idx.npy")
        if not idx.exists():
            raise ValidationError(f"Missing index file for shard {b.name}: expected {idx.name}")
        if not check_contents:
            continue
        try:
            sizes = np.load(str(idx))
        except Exception as exc:
            raise ValidationError(f"Unreadable index file {idx}: {exc}") from exc
        if sizes.ndim != 1 or sizes.size == 0:
            raise ValidationError(f"Index file {idx.name} must be a non-empty 1-D array")
        if int(sizes.astype(np.int64).sum()) != b.stat().st_size:
            raise ValidationError(
                f"Shard {b.name} is corrupt: index sums to {int(sizes.sum())} tokens but the file "
                f"holds {b.stat().st_size} bytes")
        total += int(sizes.size)
    return ShardInfo(bins, total)


def validate_pretrain_dataset(dataset_dir: str | Path) -> dict:
    root = Path(dataset_dir)
    manifest = read_manifest(root)
    validate_manifest_for_pipeline(manifest, "pretrain")
    assert isinstance(manifest, PretrainManifest)
    train = validate_pretrain_shards(root / manifest.train_dir, label="Train shard")
    val = validate_pretrain_shards(root / manifest.val_dir, label="Validation shard")
    if train["num_sequences"] != manifest.train_sequences:
        raise ValidationError(
            f"Manifest says {manifest.train_sequences} training sequences but the shards hold "
            f"{train['num_sequences']}")
    return {"manifest": manifest, "train": train, "val": val,
            "train_shards": train.paths, "val_shards": val.paths}


def _h5_files(directory: Path, prefix: str | None) -> list[Path]:
    """HDF5 shards, or their `.kdz` stand-ins (what `SaveKDDataset` writes when h5py is absent)."""
    exts = (".h5", ".kdz")
    if prefix is None:
        return sorted(f for e in exts for f in directory.glob(f"*{e}"))
    stem = Path(prefix).stem
    files = sorted(f for e in exts for f in directory.glob(f"{stem}_shard_*{e}"))
    files += [directory / (stem + e) for e in exts if (directory / (stem + e)).exists()]
    return files


def validate_hdf5_shards(directory: str | Path, prefix: str | None = None) -> dict:
    d = Path(directory)
    if not d.exists():
        raise ValidationError(f"HDF5 directory not found: {d}")
    files = _h5_files(d, prefix)
    if not files:
        raise ValidationError(f"No HDF5 files found in {d} (prefix={prefix})")
    try:
        import h5py
    except ImportError:
        return {"num_files": len(files), "num_sequences": None}
    total = 0
    for f in files:
        if f.suffix == ".kdz":
            from nanoplm_b200.data.kd_dataset import count_kd_sequences
            total += count_kd_sequences(f)
            continue
        try:
            with h5py.File(f, "r") as h:
                total += len(h.keys())
        except Exception as exc:
            raise ValidationError(f"Unreadable HDF5 file {f}: {exc}") from exc
    return {"num_files": len(files), "num_sequences": total}


def validate_distillation_dataset(dataset_dir: str | Path) -> dict:
    root = Path(dataset_dir)
    manifest = read_manifest(root)
    validate_manifest_for_pipeline(manifest, "distillation")
    assert isinstance(manifest, DistillationManifest)
    if manifest.on_the_fly:
        for key in ("train_fasta", "val_fasta"):
            p = root / getattr(manifest, key)
            if not p.exists():
                raise ValidationError(f"{key} not found: {p}")
        return {"manifest": manifest}
    train = validate_hdf5_shards(root / manifest.train_dir, manifest.train_h5_prefix)
    val = validate_hdf5_shards(root / manifest.val_dir, manifest.val_h5_prefix)
    return {"manifest": manifest, "train": train, "val": val}
