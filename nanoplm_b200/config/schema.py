"""Configuration dataclasses.

Field names and defaults follow the reference so that its YAML files load unchanged
(src/nanoplm/pretraining/config.py:8-85, src/nanoplm/pretraining/models/modern_bert/model.py:28-41,
src/nanoplm/distillation/pipeline.py:36-104, src/nanoplm/distillation/models/student/model.py:34-47).
Keys the reference does not have (conv, mHC, MoE, FP8, norm type, fused-communication switches) are
additive and default to "off".
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Optional, Union


@dataclass
class MoEConfig:
    num_experts: int = 0                 # 0 disables MoE
    top_k: int = 2
    expert_intermediate_size: int = 512
    every_n_layers: int = 2              # layers with (index % every_n_layers == every_n_layers-1) use experts
    aux_loss_coef: float = 0.01
    # expert parallelism: rows a rank's receive buffers hold, as a multiple of its even share.
    # 0 = automatic: the worst case (nothing dropped) up to 4 ranks, 4 shares beyond; rows that do not
    # fit are dropped and counted (train/moe_dropped_rows). Without expert parallelism nothing is dropped.
    capacity_factor: float = 0.0

    @property
    def enabled(self) -> bool:
        return self.num_experts > 0


@dataclass
class ModelConfig:
    """Encoder architecture. The first block of fields is the reference's ProtModernBertMLMConfig."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int = 32
    mlp_activation: str = "swiglu"
    mlp_dropout: float = 0.0
    mlp_bias: bool = False
    attention_bias: bool = False
    attention_dropout: float = 0.0
    classifier_activation: str = "gelu"
    max_position_embeddings: int = 1024
    # --- fixed in the reference's internal config (modeling.py:39-96); exposed here -------------
    hidden_activation: str = "gelu"
    initializer_range: float = 0.02      # std of the (tied) embedding / decoder initialisation
    norm_eps: float = 1e-5
    norm_bias: bool = False              # a bias vector in every norm
    classifier_bias: bool = False        # a bias in the prediction head's dense layer
    global_attn_every_n_layers: int = 3
    local_attention: int = 128
    global_rope_theta: float = 160_000.0
    local_rope_theta: float = 10_000.0
    decoder_bias: bool = True
    tie_word_embeddings: bool = True
    sparse_prediction: bool = False
    sparse_pred_ignore_index: int = -100  # label value of the positions that carry no target
    pad_token_id: int = 0
    eos_token_id: int = 1
    unk_token_id: int = 2
    mask_token_id: int = 3
    # --- additive keys ----------------------------------------------------------------------------
    embedding_dropout: float = 0.0       # after the embedding norm (fixed at 0 in the reference's config)
    norm_type: str = "layernorm"         # layernorm | rmsnorm
    conv_kernel_size: int = 0            # 0 = no conv, 7 = varlen depthwise conv before attention
    conv_bias: bool = False
    mhc_streams: int = 1                 # 1 = plain residual, 4 = hyper-connections
    mhc_sinkhorn_iters: int = 5
    moe: MoEConfig = field(default_factory=MoEConfig)

    def __post_init__(self) -> None:
        if isinstance(self.moe, dict):
            self.moe = MoEConfig(**self.moe)
        if self.moe is None:
            self.moe = MoEConfig()
        if self.hidden_size % self.num_attention_heads != 0:
            raise ValueError(
                f"hidden_size must be divisible by num_attention_heads: {self.hidden_size} vs "
                f"{self.num_attention_heads}")
        self.mlp_activation = str(self.mlp_activation).lower()
        if self.mlp_activation not in ("swiglu", "glu"):
            raise ValueError(f"Unsupported mlp_activation: {self.mlp_activation}. Supported: ['swiglu', 'glu']")
        if self.norm_type not in ("layernorm", "rmsnorm"):
            raise ValueError(f"norm_type must be layernorm or rmsnorm, got {self.norm_type}")
        if self.conv_kernel_size not in (0, 3, 5, 7, 9):
            raise ValueError("conv_kernel_size must be 0 (off) or an odd size <= 9")
        if self.mhc_streams < 1:
            raise ValueError("mhc_streams must be >= 1")
        for name in ("mlp_dropout", "attention_dropout", "embedding_dropout"):
            v = float(getattr(self, name))
            if not 0.0 <= v < 1.0:
                raise ValueError(f"{name} must be in [0, 1), got {v}")
            setattr(self, name, v)
        if self.attention_dropout > 0.0:
            # the reference drops attention probabilities inside flash-attn (dropout_p) and the
            # output projection (modeling.py:310-325, 359); the attention kernels here have no
            # probability dropout, and silently ignoring the setting would change the training recipe
            raise ValueError("attention_dropout > 0 is not supported: the varlen attention kernels implement no "
                             "dropout on attention probabilities; set attention_dropout: 0.0 "
                             "(mlp_dropout and embedding_dropout are supported)")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def sliding_window(self) -> int:
        return self.local_attention // 2

    @property
    def layer_types(self) -> list[str]:
        n = max(1, int(self.global_attn_every_n_layers))
        return ["full_attention" if i % n == 0 else "sliding_attention"
                for i in range(self.num_hidden_layers)]

    def is_moe_layer(self, i: int) -> bool:
        m = self.moe
        return m.enabled and (i % max(1, m.every_n_layers)) == max(1, m.every_n_layers) - 1


# the keys every reference pretrain.yaml must carry in its `model` section
REFERENCE_MODEL_KEYS = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
    "mlp_activation", "mlp_dropout", "mlp_bias", "attention_bias", "attention_dropout",
    "classifier_activation", "max_position_embeddings",
)


@dataclass
class PretrainingConfig:
    dataset_dir: Union[str, Path]
    ckp_dir: str = "output/pretraining"
    micro_batch_size: int = 32
    num_epochs: int = 10
    warmup_ratio: float = 0.05
    optimizer: str = "adamw"
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    adam_learning_rate: float = 1e-3
    adam_weight_decay: float = 0.0
    muon_learning_rate: float = 2e-2
    muon_weight_decay: float = 0.1
    muon_cautious_weight_decay: bool = True
    muon_use_polar_express: bool = False
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_eps: float = 1e-7
    global_batch_size: int = 2 ** 20
    bf16: bool = True
    tf32: bool = True
    mlm_probability: float = 0.3
    mask_replace_prob: float = 0.8
    random_token_prob: float = 0.1
    keep_probability: float = 0.1
    logging_steps: int = 10
    eval_steps: int = 50
    save_steps: int = 100
    seed: int = 42
    num_workers: Union[int, str] = "auto"
    prefetch_factor: int = 2
    multi_gpu: bool = False
    world_size: Union[int, str] = 1
    project_name: str = "nanoplm-pretraining"
    # --- additive keys ----------------------------------------------------------------------------
    max_grad_norm: float = 1.0
    fp8: bool = False
    fp8_recipe: str = "block128"
    expert_parallel_size: int = 1        # ranks per expert-parallel group (divides the world; every group holds all experts)
    fused_comm: bool = True              # P2P-fused reduce-scatter + AdamW + all-gather when possible
    sharded_checkpoint: bool = False     # additionally write shard-<rank>.pt + index.json
    device_masking: bool = False         # apply MLM masking on the GPU (Philox) instead of the collator
    metrics_jsonl: bool = True           # write metrics.jsonl next to the checkpoints
    heartbeat_seconds: float = 0.0       # > 0 enables the per-rank heartbeat / watchdog
    heartbeat_stall_seconds: float = 0.0  # > 0: rank 0 ends the job when a rank's step stops advancing this long
    balance_ranks: bool = True           # deal each optimizer step's sequences to ranks / micro-batches by cost
    balance_quadratic: float = 1.0 / 2700.0   # cost(len) = len + balance_quadratic * len^2
    shard_params: bool = False           # keep 1/N of every layer's weights per rank, gather inside the GEMMs
    nvtx_ranges: bool = False            # NVTX ranges around data / forward / backward / optimizer (for profilers)
    deterministic_attention: bool = False  # attention backward without atomics: bitwise reproducible, ~1.4x its time
    hf_checkpoint_files: bool = False    # also write model.safetensors + trainer_state.json (HF-Trainer layout)


@dataclass
class ResumeConfig:
    is_resume: bool = False
    checkpoint_dir: str = ""
    extra_epochs: Optional[int] = None


@dataclass
class PureTorchConfig:
    """Kept for YAML compatibility. `use_compile` is accepted and ignored: the native pipeline has no
    tracing compiler. Packing is always available; `target_packed_rows` fixes the flat batch length."""
    use_compile: bool = True
    use_packing: bool = False
    target_packed_rows: Optional[int] = None


@dataclass
class StudentConfig:
    """ProtX student (reference ProtXConfig) plus the additive architecture keys."""
    hidden_size: int = 512
    intermediate_size: int = 1024
    num_hidden_layers: int = 6
    num_attention_heads: int = 8
    # accepted for the reference's schema; the embedding table is sized from the student
    # tokenizer, as the reference does (student/model.py:59)
    vocab_size: int = 32
    mlp_activation: str = "swiglu"
    mlp_dropout: float = 0.0
    mlp_bias: bool = False
    attention_bias: bool = False
    attention_dropout: float = 0.0
    classifier_activation: str = "gelu"
    projection_layer: bool = True
    # additive
    max_position_embeddings: int = 1024
    teacher_dim: int = 1024
    norm_type: str = "layernorm"
    conv_kernel_size: int = 0
    conv_bias: bool = False
    mhc_streams: int = 1
    mhc_sinkhorn_iters: int = 5

    def to_model_config(self, vocab_size: int) -> ModelConfig:
        return ModelConfig(
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            num_hidden_layers=self.num_hidden_layers, num_attention_heads=self.num_attention_heads,
            vocab_size=vocab_size, mlp_activation=self.mlp_activation, mlp_dropout=self.mlp_dropout,
            mlp_bias=self.mlp_bias, attention_bias=self.attention_bias,
            attention_dropout=self.attention_dropout, classifier_activation=self.classifier_activation,
            max_position_embeddings=self.max_position_embeddings, norm_type=self.norm_type,
            conv_kernel_size=self.conv_kernel_size, conv_bias=self.conv_bias,
            mhc_streams=self.mhc_streams, mhc_sinkhorn_iters=self.mhc_sinkhorn_iters,
            mask_token_id=-1)


@dataclass
class TeacherConfig:
    """T5-style encoder teacher. Defaults are the ProtT5-XL encoder shape."""
    vocab_size: int = 128
    d_model: int = 1024
    d_kv: int = 128
    d_ff: int = 16384
    num_layers: int = 24
    num_heads: int = 32
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    name: str = "Rostlab/prot_t5_xl_uniref50"


@dataclass
class DistillationConfig:
    dataset_dir: Optional[Union[str, Path]] = None
    train_fasta: Optional[str] = None
    val_fasta: Optional[str] = None
    train_h5_prefix: Optional[str] = None
    val_h5_prefix: Optional[str] = None
    num_epochs: int = 10
    batch_size: int = 64
    learning_rate: float = 1e-3
    gradient_accumulation_steps: int = 1
    warmup_ratio: float = 0.05
    bf16: bool = True
    tf32: bool = True
    lr_scheduler: str = "cosine"
    lr_scheduler_kwargs: dict = field(default_factory=dict)
    max_seq_len: Optional[int] = None
    max_seqs_num: Optional[int] = None
    val_ratio: Optional[float] = None
    on_the_fly: bool = False
    sharded: bool = False
    train_sequences: Optional[int] = None
    val_sequences: Optional[int] = None
    max_open_files: int = 5
    chunk_size: int = 32
    prefetch_batches: int = 2
    use_threading: bool = True
    num_workers: int = 8
    ckp_dir: str = "output/distillation"
    project_name: str = "nanoplm-distillation"
    logging_steps: int = 10
    eval_steps: int = 50
    save_steps: int = 100
    multi_gpu: bool = False
    world_size: Union[int, str] = 1
    seed: int = 42
    # additive
    teacher: TeacherConfig = field(default_factory=TeacherConfig)
    teacher_random_init: bool = False    # benchmarks: random-init frozen teacher instead of HF weights
    max_grad_norm: float = 1.0
    fused_comm: bool = True              # P2P-fused optimizer step on multi-GPU NVLink nodes
    heartbeat_seconds: float = 0.0       # > 0 enables the per-rank heartbeat / watchdog
    heartbeat_stall_seconds: float = 0.0  # > 0: rank 0 ends the job when a rank's step stops advancing this long

    def __post_init__(self) -> None:
        if isinstance(self.teacher, dict):
            self.teacher = TeacherConfig(**self.teacher)


def field_names(cls) -> set[str]:
    return {f.name for f in fields(cls)}


def as_plain_dict(obj: Any) -> Any:
    """Dataclass -> plain nested dict (paths to str), for JSON / W&B."""
    from dataclasses import asdict, is_dataclass
    if is_dataclass(obj):
        return {k: as_plain_dict(v) for k, v in asdict(obj).items()}
    if isinstance(obj, dict):
        return {k: as_plain_dict(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [as_plain_dict(v) for v in obj]
    if isinstance(obj, Path):
        return str(obj)
    return obj
