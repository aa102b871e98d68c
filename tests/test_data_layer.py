"""FASTA preparation steps, shard round trip, manifest, validation, file pool, KD datasets."""
import gzip
import pickle
from pathlib import Path

import numpy as np
import pytest
import torch

from nanoplm_b200.data.fasta import FastaIndex, count_fasta, iter_fasta, write_fasta
from nanoplm_b200.data.file_pool import ThreadSafeFileHandlePool, detect_file_limits
from nanoplm_b200.data.manifest import (DistillationManifest, PretrainManifest, read_manifest,
                                        validate_manifest_for_pipeline, write_manifest)
from nanoplm_b200.data.prep import (Extractor, ExtractionError, FastaShuffler, Filterer, Splitor)
from nanoplm_b200.data.shards import ShardedDataset, ShardWriter
from nanoplm_b200.data.synthetic import AA_FREQ, synthetic_sequences, write_synthetic_dataset, write_synthetic_fasta
from nanoplm_b200.data.tokenizer import ProtTokenizer
from nanoplm_b200.data.validation import ValidationError, validate_pretrain_dataset, validate_pretrain_shards


def test_fasta_roundtrip_and_index(tmp_path):
    recs = [("a desc", "MKT" * 30), ("b", "ACD"), ("c", "W" * 61)]
    p = tmp_path / "x.fasta"
    write_fasta(recs, p)
    assert list(iter_fasta(p)) == recs and count_fasta(p) == 3
    idx = FastaIndex(p)
    assert len(idx) == 3 and idx.get(2) == recs[2] and idx.get(0) == recs[0]


def test_extract_filter_shuffle_split(tmp_path):
    src = write_synthetic_fasta(tmp_path / "all.fasta", 200, 5, 100, seed=1)
    gz = tmp_path / "all.fasta.gz"
    with open(src, "rb") as f, gzip.open(gz, "wb") as g:
        g.write(f.read())
    out = Extractor(gz, tmp_path / "ext.fasta").extract()
    assert out.read_bytes() == Path(src).read_bytes()
    bad = tmp_path / "bad.gz"
    bad.write_bytes(b"not gzip")
    with pytest.raises(ExtractionError):
        Extractor(bad, tmp_path / "bad.fasta").extract()
    FastaShuffler(out, tmp_path / "shuf.fasta", seed=7).shuffle()
    FastaShuffler(out, tmp_path / "shuf2.fasta", seed=7).shuffle()
    a, b = list(iter_fasta(tmp_path / "shuf.fasta")), list(iter_fasta(tmp_path / "shuf2.fasta"))
    assert a == b and a != list(iter_fasta(out)) and sorted(a) == sorted(iter_fasta(out))   # seeded permutation
    stats = Filterer(tmp_path / "shuf.fasta", tmp_path / "f.fasta", 20, 60, seqs_num=30, skip_n=5).filter()
    kept = list(iter_fasta(tmp_path / "f.fasta"))
    assert stats["kept"] == len(kept) == 30 and all(20 <= len(s) <= 60 for _, s in kept)
    n_train, n_val = Splitor(tmp_path / "f.fasta", tmp_path / "split", 0.2).split()
    assert (n_train, n_val) == (24, 6)
    assert list(iter_fasta(tmp_path / "split" / "val.fasta")) == kept[24:]


def test_synthetic_composition():
    seqs = synthetic_sequences(400, 20, 512, seed=0)
    assert all(20 <= len(s) <= 512 for s in seqs)
    text = "".join(seqs)
    freq = {a: text.count(a) / len(text) for a in AA_FREQ}
    assert abs(freq["L"] - 0.099) < 0.01 and abs(freq["W"] - 0.011) < 0.005 and set(text) <= set(AA_FREQ)


def test_shard_writer_and_dataset_roundtrip(tmp_path):
    fasta = write_synthetic_fasta(tmp_path / "t.fasta", 25, 5, 40, seed=2)
    tok = ProtTokenizer()
    w = ShardWriter(fasta, tok, max_length=32, output_dir=tmp_path / "shards", samples_per_shard=10, max_workers=2)
    shards = w.create_shards()
    assert [p.name for p in shards] == ["shard_0000.bin", "shard_0001.bin", "shard_0002.bin"]
    with pytest.raises(FileExistsError):
        ShardWriter(fasta, tok, 32, tmp_path / "shards", 10).create_shards()
    ShardWriter(fasta, tok, 32, tmp_path / "shards", 10, force=True).create_shards()
    ds = ShardedDataset(tmp_path / "shards")
    assert len(ds) == 25
    for i, (_, seq) in enumerate(iter_fasta(fasta)):
        item = ds[i]
        assert item["input_ids"].dtype == torch.uint8
        assert item["input_ids"].tolist() == tok.encode(seq, max_length=32)
        assert item["attention_mask"].all()
    with pytest.raises(IndexError):
        ds[25]
    ds2 = pickle.loads(pickle.dumps(ds))
    assert len(ds2) == 25 and ds2[3]["input_ids"].tolist() == ds[3]["input_ids"].tolist()
    assert ds.sequence_lengths().sum() == sum(len(ds[i]["input_ids"]) for i in range(25))
    with pytest.raises(FileNotFoundError):
        ShardedDataset(tmp_path / "nope")
    (tmp_path / "empty").mkdir()
    with pytest.raises(FileNotFoundError):
        ShardedDataset(tmp_path / "empty")


def test_manifest_roundtrip_and_rules(tmp_path):
    m = PretrainManifest(pipeline_mode="x", seqs_num=10, min_seq_len=5, max_seq_len=64, val_ratio=0.1,
                         train_dir="train", val_dir="val", train_sequences=9, val_sequences=1, samples_per_shard=5)
    path = write_manifest(tmp_path, m)
    assert path.name == ".data_manifest" and path.read_text().startswith("# This file is AUTO-GENERATED")
    back = read_manifest(tmp_path)
    assert isinstance(back, PretrainManifest) and back.pipeline_mode == "pretrain" and back.max_seq_len == 64
    validate_manifest_for_pipeline(back, "pretrain")
    with pytest.raises(ValueError):
        validate_manifest_for_pipeline(back, "distillation")
    with pytest.raises(ValueError):
        PretrainManifest("p", 1, 1, 1, 0.1, "a", "b", 1, 1, samples_per_shard=0)
    with pytest.raises(ValueError):
        DistillationManifest("d", 1, 1, 1, 0.1, "a", "b", 1, 1, teacher_model="prott5", on_the_fly=True)
    d = DistillationManifest("d", 1, 1, 1, 0.1, "a", "b", 1, 1, teacher_model="prott5", on_the_fly=True,
                             train_fasta="t.fasta", val_fasta="v.fasta", sharded=True, samples_per_shard=3)
    assert d.sharded is None and d.samples_per_shard is None
    with pytest.raises(FileNotFoundError):
        read_manifest(tmp_path / "missing")


def test_dataset_validation_catches_corruption(tmp_path):
    root = write_synthetic_dataset(tmp_path / "ds", 30, 6, 10, 40, samples_per_shard=10)
    info = validate_pretrain_dataset(root)
    assert info["train"] == {"num_shards": 3, "num_sequences": 30}
    (root / "train" / "shard_0001.idx.npy").rename(root / "train" / "hidden.npy")
    with pytest.raises(ValidationError, match="Missing index"):
        validate_pretrain_shards(root / "train")
    (root / "train" / "hidden.npy").rename(root / "train" / "shard_0001.idx.npy")
    with open(root / "train" / "shard_0002.bin", "ab") as f:
        f.write(b"\x05\x05")
    with pytest.raises(ValidationError, match="corrupt"):
        validate_pretrain_shards(root / "train")


class _Handle:
    def __init__(self, p):
        self.p, self.closed = p, False

    def close(self):
        self.closed = True


def _opener(p):
    return _Handle(p)


def test_file_pool_lru_hits_and_pickle(tmp_path):
    pool = ThreadSafeFileHandlePool(2, opener=_opener)
    a = pool.get("a")
    assert pool.get("a") is a
    pool.get("b")
    pool.get("c")                                 # evicts "a" (least recently used)
    assert a.closed and len(pool) == 2
    st = pool.stats()
    assert st["hits"] == 1 and st["misses"] == 3 and st["evictions"] == 1
    clone = pickle.loads(pickle.dumps(pool))
    assert len(clone) == 0 and clone.max_open_files == 2
    assert detect_file_limits(4) >= 5


def test_kd_dataset_save_load_shard(tmp_path):
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.data.kd_dataset import LoadKDDataset, SaveKDDataset, count_kd_sequences, shard_h5_file
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    fasta = write_synthetic_fasta(tmp_path / "a.fasta", 9, 8, 20, seed=3)
    teacher = T5EncoderTeacher(TeacherConfig(d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4))
    files = SaveKDDataset(fasta, tmp_path / "kd" / "train_kd.kdz", max_seq_len=24, batch_size=4, device="cpu",
                          samples_per_shard=-1, teacher=teacher).run()
    assert len(files) == 1 and count_kd_sequences(files[0]) == 9
    ds = LoadKDDataset(files[0])
    item = ds[0]
    assert item["teacher_embeddings"].shape == (24, 32) and item["input_ids"].shape == (24,)
    seq0 = next(iter_fasta(fasta))[1]
    assert int(item["attention_mask"].sum()) == len(seq0) + 1
    parts = shard_h5_file(files[0], 3, tmp_path / "kd_sharded")
    assert [count_kd_sequences(p) for p in parts] == [3, 3, 3]
    ds2 = LoadKDDataset(tmp_path / "kd_sharded" / "train_kd.kdz")
    assert len(ds2) == 9 and torch.equal(ds2[4]["teacher_embeddings"], ds[4]["teacher_embeddings"])


def test_distillation_dataset_validation(tmp_path):
    """`validate_distillation_dataset` for both forms of a distillation dataset (reference:
    data/validation.py:357-458): FASTA files of the on-the-fly form, embedding files of the stored form."""
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.data.kd_dataset import SaveKDDataset
    from nanoplm_b200.data.validation import validate_distillation_dataset, validate_hdf5_shards
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    common = dict(pipeline_mode="distillation", seqs_num=12, min_seq_len=8, max_seq_len=24, val_ratio=0.25, train_dir="train",
                  val_dir="val", train_sequences=9, val_sequences=3, teacher_model="prott5")
    fly = tmp_path / "fly"
    write_synthetic_fasta(fly / "train.fasta", 9, 8, 20, seed=1)
    write_manifest(fly, DistillationManifest(on_the_fly=True, train_fasta="train.fasta", val_fasta="val.fasta", **common))
    with pytest.raises(ValidationError, match="val_fasta not found"):
        validate_distillation_dataset(fly)
    write_synthetic_fasta(fly / "val.fasta", 3, 8, 20, seed=2)
    assert validate_distillation_dataset(fly)["manifest"].on_the_fly is True
    with pytest.raises(ValueError, match="prepared for 'distillation'"):
        validate_pretrain_dataset(fly)

    stored = tmp_path / "stored"
    teacher = T5EncoderTeacher(TeacherConfig(d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4))
    for split, n in (("train", 9), ("val", 3)):
        fasta = write_synthetic_fasta(tmp_path / f"{split}.fasta", n, 8, 20, seed=3)
        SaveKDDataset(fasta, stored / split / f"{split}_kd_dataset.kdz", max_seq_len=24, batch_size=4, device="cpu",
                      samples_per_shard=4, teacher=teacher).run()
    write_manifest(stored, DistillationManifest(on_the_fly=False, sharded=True, samples_per_shard=4,
                                                train_h5_prefix="train_kd_dataset.h5", val_h5_prefix="val_kd_dataset.h5",
                                                **common))
    info = validate_distillation_dataset(stored)
    assert info["train"]["num_files"] == 3 and info["val"]["num_files"] == 1
    assert info["train"]["num_sequences"] in (9, None)              # counted when the files can be opened
    assert validate_hdf5_shards(stored / "train")["num_files"] == 3
    with pytest.raises(ValidationError, match="No HDF5 files"):
        validate_hdf5_shards(stored / "train", prefix="other.h5")
    with pytest.raises(ValidationError, match="not found"):
        validate_hdf5_shards(stored / "nowhere")
    with pytest.raises(ValidationError, match="not a directory"):
        validate_pretrain_shards(tmp_path / "train.fasta")


def test_seqkit_backend_against_a_stand_in_binary(tmp_path, monkeypatch):
    """`FastaShuffler(backend="seqkit")` (reference: data/shuffler.py:72-95) with a stand-in `seqkit`
    that records its arguments and copies the input: the command line, a failing binary and a missing one."""
    import os
    import stat
    from nanoplm_b200.data.prep import FastaShuffler, ShufflingError
    fasta = write_synthetic_fasta(tmp_path / "in.fasta", 10, 8, 20, seed=1)
    bindir = tmp_path / "bin"
    bindir.mkdir()
    log = tmp_path / "calls.txt"
    fake = bindir / "seqkit"
    fake.write_text(f"#!/bin/sh\necho \"$@\" >> {log}\nif [ -f {tmp_path}/fail ]; then echo boom >&2; exit 2; fi\n"
                    "out=\"\"; last=\"\"\nwhile [ $# -gt 0 ]; do if [ \"$1\" = -o ]; then out=\"$2\"; shift; else last=\"$1\"; fi; shift; done\n"
                    "cp \"$last\" \"$out\"\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(bindir) + os.pathsep + os.environ["PATH"])
    out = FastaShuffler(fasta, tmp_path / "o" / "shuf.fasta", backend="seqkit", seed=11, threads=3).shuffle()
    assert out.read_bytes() == Path(fasta).read_bytes()
    words = log.read_text().split()
    assert words[0] == "shuffle" and words[words.index("--threads") + 1] == "3" and "--two-pass" in words
    assert words[words.index("--rand-seed") + 1] == "11"
    (tmp_path / "fail").write_text("")
    with pytest.raises(ShufflingError, match="boom"):
        FastaShuffler(fasta, tmp_path / "o" / "again.fasta", backend="seqkit", seed=1).shuffle()
    monkeypatch.setenv("PATH", str(tmp_path / "nothing"))
    with pytest.raises(ShufflingError, match="not on PATH"):
        FastaShuffler(fasta, tmp_path / "o" / "again.fasta", backend="seqkit", seed=1).shuffle()
    with pytest.raises(ShufflingError, match="Unknown shuffle backend"):
        FastaShuffler(fasta, tmp_path / "o" / "again.fasta", backend="sort").shuffle()
    drawn = FastaShuffler(fasta, tmp_path / "o" / "x.fasta", seed=None)
    assert 1 <= drawn.seed <= 1000                               # no seed given: one is drawn and kept


def test_kd_dataset_order_cache_pickling_and_errors(tmp_path):
    """`LoadKDDataset` (reference: distillation/dataset.py:415-781): seeded order over the shards, the
    prefetch cache returns the same items with and without threads, pickling for DataLoader workers,
    statistics, and the refusals of `SaveKDDataset` / `shard_h5_file`."""
    import pickle
    import time
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.data.kd_dataset import LoadKDDataset, SaveKDDataset, shard_h5_file
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    fasta = write_synthetic_fasta(tmp_path / "a.fasta", 23, 8, 20, seed=3)
    teacher = T5EncoderTeacher(TeacherConfig(d_model=16, d_kv=4, d_ff=32, num_layers=1, num_heads=4))
    files = SaveKDDataset(fasta, tmp_path / "kd" / "t.kdz", max_seq_len=24, batch_size=5, device="cpu",
                          samples_per_shard=6, teacher=teacher).run()
    assert [f.name for f in files] == [f"t_shard_{k:04d}.kdz" for k in range(4)]
    with pytest.raises(FileExistsError):
        SaveKDDataset(fasta, tmp_path / "kd" / "t.kdz", max_seq_len=24, device="cpu", teacher=teacher).run()
    again = SaveKDDataset(fasta, tmp_path / "kd" / "t.kdz", max_seq_len=24, batch_size=5, device="cpu", samples_per_shard=-1,
                          teacher=teacher, force=True, skip_n=3).run()
    assert len(again) == 1 and len(LoadKDDataset(again[0])) == 20 and not list((tmp_path / "kd").glob("t_shard_*"))
    with pytest.raises(FileNotFoundError):
        SaveKDDataset(tmp_path / "missing.fasta", tmp_path / "kd" / "u.kdz")
    SaveKDDataset(fasta, tmp_path / "kd" / "t.kdz", max_seq_len=24, batch_size=5, device="cpu", samples_per_shard=6,
                  teacher=teacher, force=True).run()

    plain = LoadKDDataset(tmp_path / "kd" / "t.kdz", max_open_files=2, chunk_size=4, use_threading=False)
    assert len(plain) == 23 and plain.stats()["files"] == 4 and plain.stats()["sequences"] == 23
    a = LoadKDDataset(tmp_path / "kd" / "t.kdz", chunk_size=4, seed=7)
    b = LoadKDDataset(tmp_path / "kd" / "t.kdz", chunk_size=4, seed=7, use_threading=False)
    c = LoadKDDataset(tmp_path / "kd" / "t.kdz", chunk_size=4, seed=8, use_threading=False)
    assert a._order.tolist() == b._order.tolist() != c._order.tolist() and sorted(a._order.tolist()) == list(range(23))
    for i in range(23):
        x, y = a[i], b[i]
        assert all(torch.equal(x[k], y[k]) for k in x), i
        assert torch.equal(y["input_ids"], plain[int(b._order[i])]["input_ids"])
        if i % 4 == 0:
            time.sleep(0.02)                                    # let the prefetch thread fill the cache
    with pytest.raises(IndexError):
        a[23]
    with pytest.raises(IndexError):
        a[-1]
    clone = pickle.loads(pickle.dumps(a))
    assert len(clone) == 23 and torch.equal(clone[5]["teacher_embeddings"], b[5]["teacher_embeddings"])
    with pytest.raises(FileNotFoundError):
        LoadKDDataset(tmp_path / "kd" / "nothing.kdz")
    with pytest.raises(FileNotFoundError):
        shard_h5_file(tmp_path / "kd" / "nothing.kdz", 2)
    with pytest.raises(ValueError):
        shard_h5_file(again[0] if again[0].exists() else files[0], 0)
