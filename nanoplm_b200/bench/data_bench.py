"""Host-side data pipeline throughput: shard reading, packing collators, balanced sampler.

    python -m nanoplm_b200.bench.data_bench [--sequences 40000] [--workers 0,4] [--impl reference]

`--impl reference` times the reference package's own `ShardedDataset`, `PackingCollator` and
`ProtDataCollatorForLM` (imported unmodified from `baseline/_ref`) on the same shards.

Counterpart of the reference's loading micro-benchmark (tests/shm_loading_benchmark.py:202-271 times how
fast its HDF5 shards get into shared memory; its shards are memory-mapped `.bin` + `.idx.npy` files here,
so there is no loading phase to time) for the part that matters to the training step: how many
sequences / tokens per second ONE process (and a DataLoader with workers) turns into packed, masked,
micro-batches, against what one B200 consumes with the default encoder (about 760 K real tokens per
second: `needed_tokens_per_s_per_gpu`). Needs no GPU. Prints one JSON line per measurement.
"""
from __future__ import annotations

import argparse
import json
import tempfile
import time
from pathlib import Path

import numpy as np
import torch


def _write_dataset(root: Path, n: int, lo: int, hi: int, seed: int) -> int:
    from nanoplm_b200.data.manifest import PretrainManifest, write_manifest
    from nanoplm_b200.data.synthetic import synthetic_token_sequences
    total = 0
    for split, count, s in (("train", n, seed), ("val", max(n // 50, 8), seed + 1)):
        d = root / split
        d.mkdir(parents=True, exist_ok=True)
        seqs = synthetic_token_sequences(count, lo - 1, hi - 1, s)
        if split == "train":
            total = int(sum(len(x) for x in seqs))
        per = 10000
        for i in range(0, count, per):
            part = seqs[i:i + per]
            np.concatenate(part).astype(np.uint8).tofile(d / f"shard_{i // per:04d}.bin")
            np.save(d / f"shard_{i // per:04d}.idx.npy", np.asarray([len(x) for x in part], dtype=np.int32))
    write_manifest(root, PretrainManifest(
        pipeline_mode="pretrain", seqs_num=n + max(n // 50, 8), min_seq_len=lo, max_seq_len=hi, val_ratio=0.02,
        train_dir="train", val_dir="val", train_sequences=n, val_sequences=max(n // 50, 8), sharded=True,
        samples_per_shard=10000))
    return total


def _import_reference():
    """The reference's data classes from baseline/_ref, or the reason they cannot be imported."""
    import os
    import sys
    import types
    ref_dir = Path(__file__).resolve().parents[2] / "baseline" / "_ref"
    if not (ref_dir / "nanoplm").exists():
        return "reference package not installed under baseline/_ref"
    for name, attrs in (("IPython", {"get_ipython": lambda: None}), ("h5py", {"File": object}), ("Bio", {}),
                        ("Bio.SeqIO", {})):
        try:
            __import__(name)
        except Exception:
            m = types.ModuleType(name)
            for k, v in attrs.items():
                setattr(m, k, v)
            sys.modules[name] = m
    if isinstance(sys.modules.get("Bio"), types.ModuleType) and not hasattr(sys.modules["Bio"], "SeqIO"):
        sys.modules["Bio"].SeqIO = sys.modules["Bio.SeqIO"]
    sys.path.insert(0, str(ref_dir))
    cwd = os.getcwd()
    os.chdir(tempfile.mkdtemp())           # the reference opens a log file in the current directory on import
    try:
        from nanoplm.pretraining.collator import PackingCollator, ProtDataCollatorForLM
        from nanoplm.pretraining.dataset import ShardedDataset
        from nanoplm.pretraining.models.modern_bert.tokenizer import ProtModernBertTokenizer
    except Exception as exc:
        return f"reference import failed: {type(exc).__name__}: {exc}"
    finally:
        os.chdir(cwd)
    return {"PackingCollator": PackingCollator, "ProtDataCollatorForLM": ProtDataCollatorForLM,
            "ShardedDataset": ShardedDataset, "Tokenizer": ProtModernBertTokenizer}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sequences", type=int, default=40000)
    ap.add_argument("--min-len", type=int, default=20)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--batch", type=int, default=208, help="sequences per micro-batch (the benchmark's 208)")
    ap.add_argument("--rows", type=int, default=128, help="packed rows per micro-batch")
    ap.add_argument("--workers", default="0,4", help="DataLoader worker counts to time")
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    args = ap.parse_args()

    from nanoplm_b200.data.sampler import BalancedBatchSampler
    if args.impl == "reference":
        ref = _import_reference()
        if isinstance(ref, str):
            print(json.dumps({"impl": "reference", "unavailable": ref}))
            return
        ShardedDataset, tok = ref["ShardedDataset"], ref["Tokenizer"]()
        PackingCollator = lambda t, w, p, seed=0, **kw: ref["PackingCollator"](t, w, mlm_probability=p, **kw)  # noqa: E731
        ProtDataCollatorForLM = lambda t, p, seed=0: ref["ProtDataCollatorForLM"](t, mlm_probability=p)  # noqa: E731
    else:
        from nanoplm_b200.data.collators import PackingCollator, ProtDataCollatorForLM
        from nanoplm_b200.data.shards import ShardedDataset
        from nanoplm_b200.data.tokenizer import ProtTokenizer
        tok = ProtTokenizer()
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp)
        t0 = time.perf_counter()
        tokens = _write_dataset(root, args.sequences, args.min_len, args.max_len, 7)
        print(json.dumps({"bench": "write_shards", "sequences": args.sequences, "tokens": tokens,
                          "seconds": round(time.perf_counter() - t0, 3)}), flush=True)
        ds = ShardedDataset(str(root / "train"))

        t0 = time.perf_counter()
        n_tok = 0
        for i in range(len(ds)):
            n_tok += int(ds[i]["input_ids"].numel())
        dt = time.perf_counter() - t0
        print(json.dumps({"bench": "read_every_sequence", "impl": args.impl, "sequences": len(ds), "tokens": n_tok,
                          "sequences_per_s": round(len(ds) / dt), "tokens_per_s": round(n_tok / dt)}), flush=True)

        # text -> ids, the inner loop of shard writing (pretraining/dataset.py:285-322): one call per sequence
        from nanoplm_b200.data.synthetic import synthetic_sequences
        texts = synthetic_sequences(min(args.sequences, 5000), args.min_len, args.max_len, 11)
        t0 = time.perf_counter()
        n_ids = sum(len(tok(t, add_special_tokens=True, truncation=True, max_length=args.max_len)["input_ids"])
                    for t in texts)
        dt = time.perf_counter() - t0
        print(json.dumps({"bench": "tokenize_one_by_one", "impl": args.impl, "sequences": len(texts),
                          "sequences_per_s": round(len(texts) / dt), "tokens_per_s": round(n_ids / dt)}), flush=True)

        # a B200 running the default encoder consumes about 760 K real tokens per second
        needed = 760_000
        for name, coll in (
                ("packing_collator_static", PackingCollator(tok, args.max_len, 0.3, target_rows=args.rows,
                                                            batch_size=args.batch, seed=1)),
                ("packing_collator_dynamic", PackingCollator(tok, args.max_len, 0.3, batch_size=args.batch, seed=1)),
                ("padding_collator", ProtDataCollatorForLM(tok, 0.3, seed=1))):
            for workers in [int(w) for w in args.workers.split(",")]:
                dl = torch.utils.data.DataLoader(ds, batch_size=args.batch, shuffle=False, drop_last=True,
                                                 num_workers=workers, collate_fn=coll, pin_memory=False,
                                                 persistent_workers=False)
                it = iter(dl)
                next(it)                       # worker start-up is not steady state
                t0 = time.perf_counter()
                nb = real = 0
                for b in it:
                    nb += 1
                    if "num_real_tokens" in b:
                        real += int(b["num_real_tokens"])
                    elif "attention_mask" in b:
                        real += int(b["attention_mask"].sum())
                    else:                                   # the reference's static layout: real tokens = non-pad ids
                        real += int((b["input_ids"] != 0).sum())
                dt = time.perf_counter() - t0
                print(json.dumps({"bench": name, "impl": args.impl, "workers": workers, "micro_batches": nb,
                                  "micro_batches_per_s": round(nb / dt, 1), "real_tokens_per_s": round(real / dt),
                                  "needed_tokens_per_s_per_gpu": needed,
                                  "gpus_one_loader_feeds": round(real / dt / needed, 1)}), flush=True)

        lens = np.asarray([int(ds[i]["input_ids"].numel()) for i in range(len(ds))])
        t0 = time.perf_counter()
        sampler = BalancedBatchSampler(lens, micro_batch_size=args.batch, grad_accum=2, world=8, rank=0, seed=3)
        batches = list(iter(sampler))
        dt = time.perf_counter() - t0
        print(json.dumps({"bench": "balanced_batch_sampler_epoch", "world": 8, "batches_for_rank0": len(batches),
                          "seconds": round(dt, 3)}), flush=True)


if __name__ == "__main__":
    main()
