"""Call-convention adapters: the reference's argument names and orders on top of this package's
classes and functions, for code written against `nanoplm.*` (file:line = the reference's definition).
Everything here forwards; no training logic lives in this module."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Optional, Union

import torch

from nanoplm_b200.config.schema import DistillationConfig, ModelConfig, ResumeConfig, StudentConfig
from nanoplm_b200.data import file_pool as _file_pool
from nanoplm_b200.data import kd_dataset as _kd
from nanoplm_b200.data import prep as _prep
from nanoplm_b200.data import validation as _validation
from nanoplm_b200.data.tokenizer import ProtTokenizer, StudentTokenizer
from nanoplm_b200.models.encoder import ProtEncoderMLM
from nanoplm_b200.models.student import ProtX as _ProtX
from nanoplm_b200.runtime import run_dirs as _run_dirs


# ---- models and tokenizers ------------------------------------------------------------------------
class ProtModernBertTokenizer(ProtTokenizer):
    """tokenizer.py:8-72. The special-token strings are fixed here; other values are refused."""
    _FIXED = {"unk_token": "<unk>", "pad_token": "<pad>", "eos_token": "</s>", "mask_token": "<mask>", "bos_token": "<s>"}

    def __init__(self, unk_token: str = "<unk>", pad_token: str = "<pad>", eos_token: str = "</s>",
                 mask_token: str = "<mask>", bos_token: str = "<s>", use_bos_token: bool = False, **_: Any):
        given = dict(unk_token=unk_token, pad_token=pad_token, eos_token=eos_token, mask_token=mask_token,
                     bos_token=bos_token)
        odd = {k: v for k, v in given.items() if v != self._FIXED[k]}
        if odd:
            raise ValueError(f"the special tokens of the protein vocabulary are fixed; got {odd}")
        super().__init__(use_bos_token=use_bos_token)


class ProtXTokenizer(StudentTokenizer):
    """student/tokenizer.py:4-107 (a custom `vocab` is not supported)."""

    def __init__(self, vocab: Optional[dict] = None, unk_token: str = "<unk>", pad_token: str = "<pad>",
                 eos_token: str = "</s>", **_: Any):
        if vocab is not None or (unk_token, pad_token, eos_token) != ("<unk>", "<pad>", "</s>"):
            raise ValueError("the student vocabulary and its special tokens are fixed")
        super().__init__()


class PureProtModernBertMLM(ProtEncoderMLM):
    """pure_model.py:20-46: `Model(config)`; the tokenizer is attached as `model.tokenizer`."""

    def __init__(self, config: ModelConfig):
        super().__init__(config, ProtTokenizer())

    def forward(self, *args, **kwargs):
        # the reference returns logits together with the loss; in evaluation mode so does this class
        # (in training mode they would only cost time: the training loop never reads them)
        if kwargs.get("labels") is not None and kwargs.get("return_logits") is None and not self.training:
            kwargs["return_logits"] = True
        return super().forward(*args, **kwargs)


class ProtX(_ProtX):
    """student/model.py:50-497: `ProtX(config)` and its static utilities with the reference's signatures."""

    def __init__(self, config: StudentConfig):
        super().__init__(config)

    @staticmethod
    def inspect_checkpoint_architecture(checkpoint_path: str) -> tuple[int, int, int]:
        """(embed_dim, num_layers, num_heads); the head count is a guess from the width, head size 64
        first, then 32, then 128 (student/model.py:251-354)."""
        from nanoplm_b200.models import student as S
        try:
            info = S.inspect_checkpoint_architecture(checkpoint_path)
        except Exception as exc:
            raise FileNotFoundError(f"Error loading checkpoint from {checkpoint_path}: {exc}") from exc
        h, layers = int(info["hidden_size"]), int(info["num_hidden_layers"])
        if layers == 0:
            raise ValueError("Could not determine num_layers from checkpoint")
        heads = next((h // d for d in (64, 32, 128) if h % d == 0), None)
        if heads is None:
            heads = next((n for n in (8, 12, 16, 20, 24, 32) if h % n == 0), None)
        if heads is None:
            raise ValueError("Could not determine num_heads from checkpoint")
        return h, layers, heads

    @staticmethod
    def load_and_generate_embeddings(checkpoint_path: str, sequences, batch_size: int = 32, max_length: int = 512,
                                     device: str = "cuda", per_seq_embeddings: bool = True,
                                     mlp_activation: str = "swiglu", projection_layer: bool = True):
        """Yields (sequence, embedding): pooled over the residues, or one row per residue
        (student/model.py:111-248). The architecture comes from the file."""
        from nanoplm_b200.models import student as S
        seqs = [s[:max(1, max_length - 1)] for s in sequences]
        dev = torch.device(device if (device != "cuda" or torch.cuda.is_available()) else "cpu")
        embs = S.load_and_generate_embeddings(checkpoint_path, seqs, None, batch_size=batch_size,
                                              per_token=not per_seq_embeddings, device=dev)
        yield from zip(seqs, embs)

    @staticmethod
    def _sized(embed_dim: int, num_layers: int, num_heads: int, mlp_activation: str, projection_layer: bool) -> "_ProtX":
        return _ProtX(StudentConfig(hidden_size=embed_dim, intermediate_size=4 * embed_dim, num_hidden_layers=num_layers,
                                    num_attention_heads=num_heads, mlp_activation=mlp_activation,
                                    projection_layer=projection_layer))

    @staticmethod
    def calculate_model_parameters(embed_dim: int, num_layers: int, num_heads: int, mlp_activation: str = "swiglu",
                                   projection_layer: bool = True) -> int:
        """Parameter count of a student of that shape, MLP width 4 x embed_dim (student/model.py:357-392)."""
        from nanoplm_b200.models import student as S
        return S.calculate_model_parameters(ProtX._sized(embed_dim, num_layers, num_heads, mlp_activation,
                                                         projection_layer))["total"]

    @staticmethod
    def print_parameter_breakdown(embed_dim: int, num_layers: int, num_heads: int, mlp_activation: str = "swiglu",
                                  projection_layer: bool = True) -> None:
        from nanoplm_b200.models import student as S
        S.print_parameter_breakdown(ProtX._sized(embed_dim, num_layers, num_heads, mlp_activation, projection_layer))


# ---- pretraining helpers --------------------------------------------------------------------------
def compute_batch_setup(cfg, max_seq_len: int, effective_world_size: int):
    """pretraining/utils.py:28-63."""
    return _run_dirs.compute_batch_setup(int(cfg.global_batch_size), int(cfg.micro_batch_size), int(max_seq_len),
                                         int(effective_world_size))


def prepare_run_and_steps(pretrain_config, resume_config, train_samples: int, global_batch_size_samples: int):
    """pretraining/utils.py:144-265: returns (run_name, wandb_run_name, output_dir, num_epochs,
    logging_steps, eval_steps, save_steps, resume_step)."""
    r = resume_config
    p = _run_dirs.prepare_run_and_steps(
        str(pretrain_config.ckp_dir), int(pretrain_config.num_epochs), int(pretrain_config.logging_steps),
        int(pretrain_config.eval_steps), int(pretrain_config.save_steps), bool(r and r.is_resume),
        str(r.checkpoint_dir) if r else "", getattr(r, "extra_epochs", None) if r else None, int(train_samples),
        int(global_batch_size_samples))
    return (p.run_name, p.wandb_run_name, p.output_dir, p.num_epochs, p.logging_steps, p.eval_steps, p.save_steps,
            p.resume_step)


def is_muon_optimizer(optimizer) -> bool:
    """pretraining/optim.py:10-17."""
    from nanoplm_b200.parallel.muon import is_muon_optimizer as f
    return f(optimizer)


# ---- data layer -------------------------------------------------------------------------------------
def detect_file_limits(num_workers: int = 4, reserve_percentage: float = 0.7) -> int:
    """data/file_pool.py:19-60: `reserve_percentage` is the share of the descriptor limit to use."""
    return _file_pool.detect_file_limits(num_workers, fraction=reserve_percentage)


def validate_hdf5_shards(shard_dir, expected_count: Optional[int] = None, check_contents: bool = True):
    """data/validation.py:38-179: returns the sorted shard paths."""
    _validation.validate_hdf5_shards(shard_dir)                 # existence and readability
    files = _validation._h5_files(Path(shard_dir), None)
    if expected_count is not None and len(files) != expected_count:
        raise _validation.ValidationError(f"Expected {expected_count} shard files in {shard_dir}, found {len(files)}")
    return files


class FastaShuffler(_prep.FastaShuffler):
    """data/shuffler.py:21-124 (seed before backend; seqkit always runs two-pass here)."""

    def __init__(self, input_path, output_path, seed: Optional[int] = None, backend: str = "biopython",
                 threads: int = 4, two_pass: bool = True, keep_temp: bool = False):
        super().__init__(input_path, output_path, backend=backend, seed=seed, threads=threads)


class Splitor:
    """data/splitor.py:16-54: explicit train / validation file names."""

    def __init__(self, input_file, train_file, val_file, val_ratio: float = 0.1):
        self.input_file, self.train_file, self.val_file = Path(input_file), Path(train_file), Path(val_file)
        self.val_ratio = float(val_ratio)

    def split(self) -> tuple[int, int]:
        import shutil
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            n_train, n_val = _prep.Splitor(self.input_file, tmp, self.val_ratio).split()
            for src, dst in ((Path(tmp) / "train.fasta", self.train_file), (Path(tmp) / "val.fasta", self.val_file)):
                dst.parent.mkdir(parents=True, exist_ok=True)
                shutil.move(str(src), str(dst))
        return n_train, n_val


# ---- distillation -----------------------------------------------------------------------------------
def run_distillation(model_config: StudentConfig, distill_config: DistillationConfig,
                     resume_config: Optional[ResumeConfig] = None):
    """distillation/pipeline.py:457-754."""
    from nanoplm_b200.runtime.distill import run_distillation as f
    return f(model_config, distill_config, resume_config)


class DistillDataCollator:
    """distillation/collator.py:6-111. Pre-computed mode stacks the stored tensors. On-the-fly mode
    with a `teacher_model` computes the teacher embeddings inside the collator, as the reference does;
    without one it only tokenises and leaves the teacher to the training step (this package's way)."""

    def __init__(self, teacher_model=None, teacher_tokenizer=None, student_tokenizer=None, on_the_fly: bool = False,
                 max_seq_len: int = 1024):
        from nanoplm_b200.runtime.distill import DistillDataCollator as Own
        self.teacher_model, self.on_the_fly, self.max_seq_len = teacher_model, on_the_fly, max_seq_len
        self._own = Own(on_the_fly, max_seq_len)
        if student_tokenizer is not None:
            self._own.student_tok = student_tokenizer
        if teacher_tokenizer is not None:
            self._own.teacher_tok = teacher_tokenizer

    def __call__(self, features: list) -> dict:
        batch = self._own(features)
        if not self.on_the_fly or self.teacher_model is None:
            if self.on_the_fly and self.teacher_model is None and "teacher_input_ids" not in batch:
                raise ValueError("teacher_model must be provided when on_the_fly is True.")
            return batch
        dev = next(self.teacher_model.parameters()).device
        with torch.no_grad():
            out = self.teacher_model(batch["teacher_input_ids"].to(dev), batch["teacher_attention_mask"].to(dev))
        emb = getattr(out, "last_hidden_state", out)
        return {"input_ids": batch["input_ids"], "attention_mask": batch["attention_mask"],
                "teacher_embeddings": emb.cpu().float()}


class KDDatasetOnTheFly(_kd.KDDatasetOnTheFly):
    """distillation/dataset.py:21-52 (the teacher, device and read batch size play no part here)."""

    def __init__(self, input_fasta, teacher=None, max_seq_len: Optional[int] = None, device: Optional[str] = None,
                 read_batch_size: Optional[int] = None):
        super().__init__(input_fasta)


class SaveKDDataset(_kd.SaveKDDataset):
    """distillation/dataset.py:55-412: `process_dataset()` returns one path or the list of shards."""

    def __init__(self, input_fasta, output_path, teacher=None, mode: str = "get_embeddings", max_seq_len: int = 1024,
                 batch_size: int = 4, device: str = "auto", skip_n: int = 0, samples_per_shard: int = -1,
                 force: bool = False):
        if mode != "get_embeddings":
            raise ValueError(f"unsupported mode {mode!r}: embeddings are always computed")
        super().__init__(input_fasta, output_path, max_seq_len=max_seq_len, batch_size=batch_size, device=device,
                         samples_per_shard=samples_per_shard, teacher=teacher, force=force, skip_n=skip_n)

    def process_dataset(self) -> Union[Path, list]:
        files = self.run()
        return files if self.samples_per_shard > 0 else files[0]


class LoadKDDataset(_kd.LoadKDDataset):
    """distillation/dataset.py:415-781 (items are host tensors; `device` is accepted and unused)."""

    def __init__(self, h5_path, device: Optional[str] = None, seed: Optional[int] = None,
                 sharded: Optional[bool] = None, max_open_files: int = 5, chunk_size: int = 32,
                 prefetch_batches: int = 2, use_threading: bool = True):
        super().__init__(h5_path, max_open_files, chunk_size, prefetch_batches, use_threading, seed=seed,
                         sharded=sharded)


def shard_h5_file(input_h5_path, n_sharded_files: int, output_dir=None, total_sequences: Optional[int] = None):
    """distillation/dataset.py:784-906."""
    return _kd.shard_h5_file(input_h5_path, n_sharded_files, output_dir, total_sequences)


# ---- utilities --------------------------------------------------------------------------------------
def read_yaml(file_path):
    """utils/common.py:30-39."""
    from nanoplm_b200.config.loaders import read_yaml as f
    return f(file_path)


def log_stage(stage_name: str) -> None:
    """utils/logger.py:31-33."""
    from nanoplm_b200.utils.logging import log_stage as f
    f(stage_name)


def create_dirs(path) -> None:
    """utils/common.py:52-59: a path with a file extension names a file (its parent is created)."""
    d = Path(path)
    d = d.parent if d.suffix else d
    d.mkdir(parents=True, exist_ok=True)


def get_device() -> str:
    """utils/common.py: "cuda" when a GPU is visible, else "cpu"."""
    return "cuda" if torch.cuda.is_available() else "cpu"


def is_flash_attention_available() -> bool:
    """utils/common.py:16-27: whether the fast varlen attention path can run. Here that is this
    package's own kernels, which need a CUDA device."""
    return torch.cuda.is_available()


def inside_git_repo(work_dir) -> bool:
    """utils/common.py:112-130."""
    from nanoplm_b200.cli.data import _inside_git_repo
    return _inside_git_repo(Path(work_dir))


def is_git_subdir(work_dir) -> bool:
    """utils/common.py:143-165."""
    from nanoplm_b200.cli.data import _is_git_subdir
    return _is_git_subdir(Path(work_dir))


def get_caller_dir() -> Path:
    """utils/common.py:61-109: the directory relative paths are resolved against, i.e. the working
    directory (the reference walks the call stack to the same effect for command-line use)."""
    return Path.cwd()
