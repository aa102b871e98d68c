"""`nanoplm data ...`: dataset download / preparation commands (reference: src/nanoplm/cli/data.py).

Sub-commands and options match the reference. `from-yaml` runs the stages of `params.yaml`
(download -> extract -> shuffle -> filter -> split [-> save-kd-dataset x2]) and then writes the
binary shards / the `.data_manifest`. The reference delegates stage execution to the external `dvc`
binary; here the stages also run in-process (`--runner builtin`, the default when `dvc` is not
installed) with the same inputs, outputs and skip-if-up-to-date behaviour, so data preparation
works on machines without DVC.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

import click

from nanoplm_b200.config.datasets import DATASET_URLS, resolve_dataset_url
from nanoplm_b200.config.loaders import read_yaml
from nanoplm_b200.config.templates import DVC_YAML, PARAMS_YAML
from nanoplm_b200.data.fasta import count_fasta
from nanoplm_b200.data.manifest import DistillationManifest, PretrainManifest, write_manifest
from nanoplm_b200.data.prep import (DownloadError, Downloader, ExtractionError, Extractor, FastaShuffler,
                                    FilterError, Filterer, ShufflingError, SplitError, Splitor)


@click.group(help="Group of commands for dataset download and preparation.")
def data() -> None:
    pass


def _make_dirs(path: Path) -> None:
    """A path with a file extension names a file (its parent is created), any other a directory
    (reference: utils/common.py:52-59)."""
    d = Path(path)
    d = d.parent if d.suffix else d
    d.mkdir(parents=True, exist_ok=True)


def _resolve(p, cwd: Path) -> Path:
    p = Path(p)
    return p if p.is_absolute() else cwd / p


# ----------------------------------------------------------------------------------- simple steps
@data.command("download", help="Download a dataset by key (see --help for keys) or from --url.")
@click.argument("dataset", required=False, type=click.Choice(sorted(DATASET_URLS), case_sensitive=False))
@click.option("--url", default=None, help="Explicit download URL (instead of a dataset key).")
@click.option("-o", "--output", "output", default="downloaded_dataset", show_default=True,
              type=click.Path(path_type=Path), help="Target file, or a directory (the file keeps the URL's name).")
@click.option("-f", "--force", is_flag=True, help="Overwrite an existing file.")
def download(dataset, url, output: Path, force: bool) -> None:
    if not dataset and not url:
        raise click.UsageError("Either a dataset key or --url must be provided.")
    if dataset and url:
        raise click.UsageError("Both a dataset key and --url cannot be provided.")
    try:
        src = resolve_dataset_url(dataset, url)
    except KeyError as exc:
        raise click.ClickException(str(exc).strip("'\"")) from exc
    _make_dirs(output)
    if output.is_dir():
        output = output / Path(src).name
    if output.exists():
        if not force:
            # the reference reports and leaves with exit code 0 (cli/data.py:96-105)
            click.echo(f"File already exists: {output} \nUse --force to overwrite.")
            return
        output.unlink()
    try:
        Downloader(src, output).download()
    except DownloadError as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Downloaded {src} -> {output}")


@data.command("extract", help="Decompress a .gz FASTA file.")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "output", required=True, type=click.Path(path_type=Path))
@click.option("-f", "--force", is_flag=True)
def extract(input_path: Path, output: Path, force: bool) -> None:
    if output.exists() and not force:
        raise click.ClickException(f"Output already exists: {output}. Use --force to overwrite.")
    try:
        Extractor(input_path, output).extract()
    except ExtractionError as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Extracted {input_path} -> {output}")


@data.command("shuffle", help="Shuffle the records of a FASTA file.")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "output", required=True, type=click.Path(path_type=Path))
@click.option("--backend", type=click.Choice(["seqkit", "biopython"]), default="biopython")
@click.option("--seed", type=int, default=None, help="Random seed (none: a different order every run).")
def shuffle(input_path: Path, output: Path, backend: str, seed: int) -> None:
    if input_path.suffix != ".fasta":
        raise click.ClickException("Input file must have a .fasta extension")
    try:
        FastaShuffler(input_path, output, backend=backend, seed=seed).shuffle()
    except ShufflingError as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Shuffled {input_path} -> {output}")


@data.command("filter", help="Keep sequences within a length range, up to a maximum count.")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "output", required=True, type=click.Path(path_type=Path))
@click.option("--min-seq-len", type=int, default=20)
@click.option("--max-seq-len", type=int, default=1024)
@click.option("--seqs-num", type=int, default=-1, help="-1 keeps every matching sequence.")
@click.option("--skip-n", type=int, default=0)
def filter_cmd(input_path, output, min_seq_len, max_seq_len, seqs_num, skip_n) -> None:
    try:
        stats = Filterer(input_path, output, min_seq_len, max_seq_len, seqs_num, skip_n).filter()
    except FilterError as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Filtered {stats['kept']} of {stats['processed']} sequences -> {output}")


@data.command("split", help="Split a FASTA file into train.fasta and val.fasta.")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "--output-dir", "output_dir", required=True, type=click.Path(path_type=Path),
              help="Directory that receives train.fasta and val.fasta.")
@click.option("--val-ratio", type=float, default=0.1)
def split(input_path, output_dir, val_ratio) -> None:
    try:
        n_train, n_val = Splitor(input_path, output_dir, val_ratio).split()
    except SplitError as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Split into {n_train} train / {n_val} val sequences -> {output_dir}")


@data.command("save-pretrain-dataset", help="Tokenise a FASTA file into binary shards (.bin + .idx.npy).")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "--output-dir", "output_dir", required=True, type=click.Path(path_type=Path))
@click.option("--max-seq-len", type=int, default=1024)
@click.option("--samples-per-shard", type=int, default=10000)
@click.option("--max-workers", type=int, default=2, help="-1 uses every CPU.")
@click.option("-f", "--force", is_flag=True)
def save_pretrain_dataset(input_path, output_dir, max_seq_len, samples_per_shard, max_workers, force) -> None:
    from nanoplm_b200.data.shards import ShardWriter
    from nanoplm_b200.data.tokenizer import ProtTokenizer
    try:
        w = ShardWriter(input_path, ProtTokenizer(), max_seq_len, output_dir, samples_per_shard, max_workers, force)
        shards = w.create_shards()
    except (FileNotFoundError, FileExistsError, ValueError) as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Wrote {len(shards)} shards ({len(w)} sequences) -> {output_dir}")


@data.command("save-kd-dataset", help="Compute teacher embeddings for a FASTA file and store them (HDF5).")
@click.option("-i", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-o", "--output", "output", required=True, type=click.Path(path_type=Path))
@click.option("--teacher-model", default="prott5")
@click.option("--max-seq-len", type=int, default=1024)
@click.option("--batch-size", type=int, default=4)
@click.option("--device", default="auto", type=click.Choice(["auto", "cuda", "mps", "cpu"]))
@click.option("--samples-per-shard", type=int, default=-1, help="-1 writes a single file.")
@click.option("--skip-n", type=int, default=0, help="Skip the first n sequences of the input.")
@click.option("--teacher-random-init", is_flag=True, help="Random-init teacher (offline machines, tests).")
@click.option("-f", "--force", is_flag=True)
def save_kd_dataset(input_path, output, teacher_model, max_seq_len, batch_size, device, samples_per_shard,
                    skip_n, teacher_random_init, force) -> None:
    if teacher_model.lower() != "prott5":
        raise click.ClickException(f"Teacher model {teacher_model} not supported")
    if samples_per_shard < -1 or samples_per_shard == 0:
        raise click.ClickException("samples-per-shard must be -1 (no sharding) or a positive number (not 0)")
    if batch_size < 1:
        raise click.ClickException("batch-size must be at least 1")
    if max_seq_len < 1:
        raise click.ClickException("max-seq-len must be at least 1")
    if skip_n < 0:
        raise click.ClickException("skip-n must be at least 0")
    from nanoplm_b200.data.kd_dataset import SaveKDDataset, have_h5py
    output = Path(output)
    _make_dirs(output)
    if output.is_dir():
        ext = ".h5" if have_h5py() else ".kdz"
        output = output / Path(input_path).name.replace(".fasta", "_kd_dataset" + ext)
    elif output.suffix not in (".h5", ".kdz"):
        raise click.ClickException("Output must end with .h5 (.kdz without h5py) or be a directory")
    try:
        saver = SaveKDDataset(input_path, output, max_seq_len=max_seq_len, batch_size=batch_size, device=device,
                              samples_per_shard=samples_per_shard, random_init_teacher=teacher_random_init,
                              force=force, skip_n=skip_n)
        files = saver.run()
    except (FileNotFoundError, FileExistsError, ValueError, RuntimeError) as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Wrote {len(files)} file(s) -> {Path(output).parent}")


@data.command("shard", help="Split one large KD dataset file into n shards.")
@click.option("-i", "--input-file", "--input", "input_path", required=True, type=click.Path(path_type=Path))
@click.option("-n", "--n-shards", "--num-shards", "n", required=True, type=int)
@click.option("-o", "--output-dir", "output_dir", default=None, type=click.Path(path_type=Path))
@click.option("-t", "--total-sequences", "--total", "total", default=None, type=int,
              help="Total number of sequences (skips counting).")
def shard(input_path, n, output_dir, total) -> None:
    from nanoplm_b200.data.kd_dataset import shard_h5_file
    try:
        files = shard_h5_file(input_path, n, output_dir, total)
    except (FileNotFoundError, ValueError, RuntimeError) as exc:
        raise click.ClickException(str(exc)) from exc
    click.echo(f"Wrote {len(files)} shards")


# ----------------------------------------------------------------------------------- templates
@data.command("get-yaml", help="Write params.yaml and dvc.yaml templates.")
@click.argument("output", required=False, type=click.Path(path_type=Path))
@click.option("--force", is_flag=True)
def get_yaml(output, force) -> None:
    out_dir = Path.cwd() if output is None else Path(output)
    out_dir.mkdir(parents=True, exist_ok=True)
    for name, text in (("params.yaml", PARAMS_YAML), ("dvc.yaml", DVC_YAML)):
        target = out_dir / name
        if target.exists() and not force:
            raise click.ClickException(f"File already exists: {target}. Use --force to overwrite.")
        target.write_text(text, encoding="utf-8")
        click.echo(f"Template written to: {target}")


# ----------------------------------------------------------------------------------- from-yaml
def _stale(outputs: list[Path], inputs: list[Path]) -> bool:
    if not all(o.exists() for o in outputs):
        return True
    newest_in = max((i.stat().st_mtime for i in inputs if i.exists()), default=0.0)
    return any(o.stat().st_mtime < newest_in for o in outputs)


def run_builtin_stages(params: dict, cwd: Path, upto: str | None, force: bool) -> None:
    """In-process equivalent of `dvc repro [target]` for the stages of the dvc.yaml template."""
    dp, dd = params.get("data_params", {}), params.get("data_dirs", {})
    comp, ext = _resolve(dd["compressed_fasta"], cwd), _resolve(dd["extracted_fasta"], cwd)
    shuf, filt = _resolve(dd["shuffled_fasta"], cwd), _resolve(dd["filtered_fasta"], cwd)
    split_dir = _resolve(dd["splitted_fasta_dir"], cwd)

    def stage_download():
        if not ext.exists() and (force or not comp.exists()):
            click.echo("[download]")
            Downloader(dd["url"], comp).download()

    def stage_extract():
        if force or (comp.exists() and _stale([ext], [comp])):
            click.echo("[extract]")
            Extractor(comp, ext).extract()

    def stage_shuffle():
        if not dp.get("shuffle", True):
            if force or _stale([shuf], [ext]):
                shuf.parent.mkdir(parents=True, exist_ok=True)
                shutil.copyfile(ext, shuf)
            return
        if force or _stale([shuf], [ext]):
            click.echo("[shuffle]")
            FastaShuffler(ext, shuf, dp.get("shuffle_backend", "biopython"), dp.get("shuffle_seed", 24)).shuffle()

    def stage_filter():
        if force or _stale([filt], [shuf]):
            click.echo("[filter]")
            Filterer(shuf, filt, dp.get("min_seq_len", 20), dp.get("max_seq_len", 512), dp.get("seqs_num", -1),
                     dp.get("filter_skip_n", 0)).filter()

    def stage_split():
        outs = [split_dir / "train.fasta", split_dir / "val.fasta"]
        if force or _stale(outs, [filt]):
            click.echo("[split]")
            Splitor(filt, split_dir, dp.get("val_ratio", 0.1)).split()

    def stage_kd(which: str):
        from nanoplm_b200.data.kd_dataset import SaveKDDataset
        dc = params.get("distillation_config", {})
        out = _resolve(dc.get("output_dir", "output/data/kd_dataset"), cwd) / which / f"{which}_kd_dataset.h5"
        src = split_dir / f"{which}.fasta"
        if force or _stale([out.parent], [src]) or not any(out.parent.glob("*")):
            click.echo(f"[save_kd_{which}_dataset]")
            SaveKDDataset(src, out, max_seq_len=dp.get("max_seq_len", 512),
                          batch_size=dc.get("embed_calc_batch_size", 4), device=dp.get("device", "auto"),
                          samples_per_shard=dc.get("samples_per_shard", -1),
                          random_init_teacher=bool(dc.get("teacher_random_init", False)), force=True).run()

    stages = [("download", stage_download), ("extract", stage_extract), ("shuffle", stage_shuffle),
              ("filter", stage_filter), ("split", stage_split),
              ("save_kd_train_dataset", lambda: stage_kd("train")),
              ("save_kd_val_dataset", lambda: stage_kd("val"))]
    names = [n for n, _ in stages]
    if upto is not None and upto not in names:
        raise click.ClickException(f"Unknown target stage '{upto}'. Stages: {', '.join(names)}")
    for name, fn in stages:
        fn()
        if name == upto:
            break


def _inside_git_repo(path: Path) -> bool:
    try:
        r = subprocess.run(["git", "rev-parse", "--is-inside-work-tree"], cwd=str(path), capture_output=True, text=True)
        return r.returncode == 0 and r.stdout.strip() == "true"
    except FileNotFoundError:
        return False


def _is_git_subdir(path: Path) -> bool:
    try:
        r = subprocess.run(["git", "rev-parse", "--show-toplevel"], cwd=str(path), capture_output=True, text=True)
        return r.returncode == 0 and Path(r.stdout.strip()).resolve() != path.resolve()
    except FileNotFoundError:
        return False


def _count_sequences_in_dir(d: Path) -> int:
    from nanoplm_b200.data.kd_dataset import count_kd_sequences
    return sum(count_kd_sequences(f) for f in sorted(d.glob("*.h5")) + sorted(d.glob("*.kdz")))


def _h5_prefix(files: list[Path], default: str) -> str:
    if not files:
        return default
    name = sorted(files)[0].name
    if "_shard_" in name:
        return name.split("_shard_")[0] + Path(name).suffix
    return name


@data.command("from-yaml", help="Run the data preparation pipeline described by params.yaml.")
@click.argument("config", default="params.yaml", type=click.Path(dir_okay=False, path_type=Path))
@click.option("--target", default=None, help="Run the pipeline only up to this stage.")
@click.option("--no-auto-init", is_flag=True, help="Do not run `dvc init` automatically (dvc runner).")
@click.option("--force", "force_repro", is_flag=True, help="Re-run stages even when up to date.")
@click.option("--verbose", is_flag=True)
@click.option("--runner", type=click.Choice(["auto", "dvc", "builtin"]), default="auto",
              help="Stage executor: the external dvc binary or the built-in runner.")
def from_yaml(config: Path, target, no_auto_init, force_repro, verbose, runner) -> None:
    params_yaml = config if config.is_absolute() else Path.cwd() / config
    cwd = params_yaml.parent
    if not params_yaml.exists():
        raise click.ClickException(f"params.yaml not found in {cwd}.\nUse `nanoplm data get-yaml` to "
                                   "generate a params.yaml file.")
    try:
        params = read_yaml(params_yaml)
    except Exception as exc:  # noqa: BLE001
        raise click.ClickException(f"Failed to read params.yaml: {exc}") from exc
    dp = params.get("data_params", {}) or {}
    mode = dp.get("pipeline_mode", "pretrain")
    if mode not in ("none", "pretrain", "distillation"):
        raise click.ClickException(f"Invalid pipeline_mode: '{mode}'. Must be one of: distillation, none, pretrain")
    dc = params.get("distillation_config", {}) or {}
    on_the_fly = bool(dc.get("on_the_fly", False))
    if target is None and not (mode == "distillation" and not on_the_fly):
        target = "split"
    click.echo(f"Running pipeline{' up to ' + repr(target) if target else ''} (pipeline_mode: '{mode}')")

    use_dvc = runner == "dvc" or (runner == "auto" and shutil.which("dvc") is not None
                                  and (cwd / "dvc.yaml").exists())
    if use_dvc:
        if shutil.which("dvc") is None:
            raise click.ClickException("'dvc' command not found. Please install DVC (pip install dvc).")
        if not (cwd / ".dvc").exists():
            if no_auto_init:
                raise click.ClickException(f"DVC is not initialized in {cwd}. Run 'dvc init' first.")
            init = ["dvc", "init", "-q"]
            if not _inside_git_repo(cwd):
                init.append("--no-scm")
            elif _is_git_subdir(cwd):
                init.append("--subdir")
            subprocess.run(init, cwd=str(cwd), check=True)
        cmd = ["dvc", "repro"] + (["-v"] if verbose else []) + (["-f"] if force_repro else [])
        if target:
            cmd.append(target)
        try:
            subprocess.run(cmd, cwd=str(cwd), check=True)
        except subprocess.CalledProcessError as exc:
            raise click.ClickException(f"dvc repro failed with exit code {exc.returncode}") from exc
    else:
        try:
            run_builtin_stages(params, cwd, target, force_repro)
        except (DownloadError, ExtractionError, ShufflingError, FilterError, SplitError, KeyError) as exc:
            raise click.ClickException(f"data stage failed: {exc}") from exc

    dd = params.get("data_dirs", {}) or {}
    split_dir = dd.get("splitted_fasta_dir")
    if mode == "pretrain":
        from nanoplm_b200.data.shards import ShardWriter
        from nanoplm_b200.data.tokenizer import ProtTokenizer
        if not split_dir:
            raise click.ClickException("data_dirs.splitted_fasta_dir is required for pretrain mode")
        pc = params.get("pretrain_config", {}) or {}
        out = _resolve(pc.get("output_dir", "output/data/pretrain_shards"), cwd)
        tok = ProtTokenizer()
        counts = {}
        for which in ("train", "val"):
            click.echo(f"Creating binary shards for {which} dataset...")
            try:
                w = ShardWriter(_resolve(Path(split_dir) / f"{which}.fasta", cwd), tok, dp.get("max_seq_len"),
                                out / which, pc.get("samples_per_shard", 10000), pc.get("max_workers", -1),
                                bool(pc.get("force", False)) or force_repro)
                shards = w.create_shards()
            except (FileNotFoundError, FileExistsError, ValueError) as exc:
                raise click.ClickException(str(exc)) from exc
            counts[which] = (len(shards), len(w))
        path = write_manifest(out, PretrainManifest(
            pipeline_mode="pretrain", seqs_num=dp.get("seqs_num"), min_seq_len=dp.get("min_seq_len"),
            max_seq_len=dp.get("max_seq_len"), val_ratio=dp.get("val_ratio"), train_dir="train", val_dir="val",
            train_sequences=counts["train"][1], val_sequences=counts["val"][1], sharded=True,
            samples_per_shard=pc.get("samples_per_shard", 10000)))
        click.echo("Pretraining shard generation complete:\n"
                   f"  Train shards: {counts['train'][0]} ({counts['train'][1]} sequences) -> {out / 'train'}\n"
                   f"  Val shards:   {counts['val'][0]} ({counts['val'][1]} sequences) -> {out / 'val'}\n"
                   f"  Manifest: {path}")
    elif mode == "distillation":
        out = _resolve(dc.get("output_dir", "output/data/kd_dataset"), cwd)
        common = dict(pipeline_mode="distillation", seqs_num=dp.get("seqs_num"), min_seq_len=dp.get("min_seq_len"),
                      max_seq_len=dp.get("max_seq_len"), val_ratio=dp.get("val_ratio"), train_dir="train",
                      val_dir="val", teacher_model=dc.get("teacher_model", "prott5"))
        if on_the_fly:
            if not split_dir:
                raise click.ClickException("data_dirs.splitted_fasta_dir is required for distillation mode")
            tr, va = _resolve(Path(split_dir) / "train.fasta", cwd), _resolve(Path(split_dir) / "val.fasta", cwd)
            path = write_manifest(out, DistillationManifest(
                **common, train_sequences=count_fasta(tr), val_sequences=count_fasta(va), on_the_fly=True,
                train_fasta=str(tr), val_fasta=str(va)))
            click.echo(f"Distillation manifest created (on-the-fly mode): {path}")
        else:
            sps = int(dc.get("samples_per_shard", -1))
            tr_files = sorted((out / "train").glob("*.h5")) + sorted((out / "train").glob("*.kdz"))
            va_files = sorted((out / "val").glob("*.h5")) + sorted((out / "val").glob("*.kdz"))
            path = write_manifest(out, DistillationManifest(
                **common, train_sequences=_count_sequences_in_dir(out / "train"),
                val_sequences=_count_sequences_in_dir(out / "val"), sharded=True,
                samples_per_shard=sps if sps > 0 else max(1, _count_sequences_in_dir(out / "train")),
                train_h5_prefix=_h5_prefix(tr_files, "train_kd_dataset.h5"),
                val_h5_prefix=_h5_prefix(va_files, "val_kd_dataset.h5"), on_the_fly=False))
            click.echo(f"Distillation dataset generation complete. Manifest: {path}")
    else:
        click.echo("Data preparation complete (pipeline_mode: 'none')")
