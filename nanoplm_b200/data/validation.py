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


def validate_pretrain_shards(shard_dir: str | Path, label: str = "shards") -> dict:
    d = Path(shard_dir)
    if not d.exists():
        raise ValidationError(f"{label} directory not found: {d}")
    bins = sorted(d.glob("*.bin"))
    if not bins:
        raise ValidationError(f"No binary shard files (*.bin) found in {d}")
    total = 0
    for b in bins:
        idx = b.with_name(b.stem + ".idx.npy")
        if not idx.exists():
            raise ValidationError(f"Missing index file for shard {b.name}: expected {idx.name}")
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
    return {"num_shards": len(bins), "num_sequences": total}


def validate_pretrain_dataset(dataset_dir: str | Path) -> dict:
    root = Path(dataset_dir)
    manifest = read_manifest(root)
    validate_manifest_for_pipeline(manifest, "pretrain")
    assert isinstance(manifest, PretrainManifest)
    train = validate_pretrain_shards(root / manifest.train_dir, "Train shard")
    val = validate_pretrain_shards(root / manifest.val_dir, "Validation shard")
    if train["num_sequences"] != manifest.train_sequences:
        raise ValidationError(
            f"Manifest says {manifest.train_sequences} training sequences but the shards hold "
            f"{train['num_sequences']}")
    return {"manifest": manifest, "train": train, "val": val}


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
