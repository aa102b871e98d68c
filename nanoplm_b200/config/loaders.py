"""YAML section -> dataclass loaders with strict key checking and string coercion.

Contract (reference: src/nanoplm/cli/pretrain.py:704-924, src/nanoplm/cli/distill.py:629-743):
  * `model` (pretrain): every reference key is required, unknown keys are rejected; the additive
    keys of this framework are optional.
  * `pretraining`: `dataset_dir` required; `learning_rate` / `weight_decay` are accepted as
    deprecated aliases; `gradient_accumulation_steps` is rejected (it is inferred); unknown keys
    rejected; numbers written as strings ("1e-3") and booleans written as strings are coerced.
  * `pure_torch`: {enabled, use_compile, use_packing, target_packed_rows}.
  * `resume`: {is_resume, checkpoint_dir, extra_epochs}; resuming from a missing directory fails.
"""
from __future__ import annotations

import logging
from dataclasses import fields
from pathlib import Path
from typing import Any, Mapping, Optional

from .schema import (REFERENCE_MODEL_KEYS, DistillationConfig, ModelConfig, MoEConfig,
                     PretrainingConfig, PureTorchConfig, ResumeConfig, StudentConfig, TeacherConfig,
                     field_names)

log = logging.getLogger("nanoplm_b200")


class ConfigError(ValueError):
    pass


def _to_bool(v: Any, key: str) -> bool:
    if isinstance(v, bool):
        return v
    if isinstance(v, str):
        s = v.strip().lower()
        if s in ("true", "yes", "1", "on"):
            return True
        if s in ("false", "no", "0", "off", ""):
            return False
    if isinstance(v, (int, float)):
        return bool(v)
    raise ConfigError(f"Invalid boolean for {key}: {v!r}")


def _to_float(v: Any, key: str) -> float:
    try:
        return float(v)
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"Invalid {key} value: {v}. Must be a number.") from exc


def _to_int(v: Any, key: str) -> int:
    if isinstance(v, bool):
        raise ConfigError(f"Invalid {key} value: {v}. Must be an integer.")
    try:
        f = float(v)
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"Invalid {key} value: {v}. Must be an integer.") from exc
    if f != int(f):
        raise ConfigError(f"Invalid {key} value: {v}. Must be an integer.")
    return int(f)


def _coerce(cls, kwargs: dict) -> dict:
    """Coerces values to the annotated scalar type of each dataclass field."""
    out = dict(kwargs)
    for f in fields(cls):
        if f.name not in out or out[f.name] is None:
            continue
        ann = str(f.type)
        v = out[f.name]
        if ann in ("bool", "<class 'bool'>"):
            out[f.name] = _to_bool(v, f.name)
        elif ann in ("float", "<class 'float'>"):
            out[f.name] = _to_float(v, f.name)
        elif ann in ("int", "<class 'int'>"):
            out[f.name] = _to_int(v, f.name)
        elif ann.startswith("Optional[int") and not isinstance(v, int):
            out[f.name] = _to_int(v, f.name)
        elif ann.startswith("Optional[float") and not isinstance(v, float):
            out[f.name] = _to_float(v, f.name)
    return out


def load_model_config(section: Optional[Mapping[str, Any]]) -> ModelConfig:
    if section is None:
        raise ConfigError("Model configuration is required but not found in YAML")
    known = field_names(ModelConfig)
    extra = sorted(k for k in section if k not in known)
    missing = sorted(k for k in REFERENCE_MODEL_KEYS if section.get(k) is None)
    if missing:
        raise ConfigError(f"Missing required model configuration keys: {', '.join(missing)}")
    if extra:
        raise ConfigError(f"Unexpected model configuration keys: {', '.join(extra)}")
    kwargs = {k: v for k, v in section.items() if v is not None}
    if isinstance(kwargs.get("moe"), Mapping):
        moe_known = field_names(MoEConfig)
        bad = sorted(k for k in kwargs["moe"] if k not in moe_known)
        if bad:
            raise ConfigError(f"Unexpected model.moe keys: {', '.join(bad)}")
        kwargs["moe"] = MoEConfig(**_coerce(MoEConfig, dict(kwargs["moe"])))
    return ModelConfig(**_coerce(ModelConfig, kwargs))


_LEGACY_ALIASES = {"learning_rate": "adam_learning_rate", "weight_decay": "adam_weight_decay"}


def load_pretrain_config(section: Optional[Mapping[str, Any]]) -> PretrainingConfig:
    if section is None:
        raise ConfigError("Pretraining configuration is required but not found in YAML")
    cfg = dict(section)
    for old, new in _LEGACY_ALIASES.items():
        if old not in cfg:
            continue
        old_v, new_v = cfg.pop(old), cfg.get(new)
        if old_v is None:
            continue
        if new_v is None:
            cfg[new] = old_v
            log.warning("Deprecated key '%s' detected; please use '%s' instead.", old, new)
        else:
            try:
                same = float(old_v) == float(new_v)
            except (TypeError, ValueError):
                same = old_v == new_v
            if not same:
                log.warning("Both '%s' and '%s' are set with different values. Using '%s' and "
                            "ignoring '%s'.", old, new, new, old)
    if "gradient_accumulation_steps" in cfg:
        raise ConfigError(
            "gradient_accumulation_steps is inferred automatically from global_batch_size, "
            "micro_batch_size, max_seq_len, and world_size. Remove gradient_accumulation_steps "
            "from your pretraining config.")
    if not cfg.get("dataset_dir"):
        raise ConfigError("dataset_dir is required in pretraining configuration")
    known = field_names(PretrainingConfig)
    extra = sorted(k for k in cfg if k not in known)
    if extra:
        raise ConfigError(f"Unexpected training configuration keys: {', '.join(extra)}")
    kwargs = {k: v for k, v in cfg.items() if v is not None}
    return PretrainingConfig(**_coerce(PretrainingConfig, kwargs))


def resolve_pure_torch_config(raw: Mapping[str, Any]) -> tuple[bool, PureTorchConfig]:
    """Returns (enabled, PureTorchConfig) from the optional `pure_torch` section."""
    sec = raw.get("pure_torch")
    if not isinstance(sec, Mapping):
        return False, PureTorchConfig()
    enabled = _to_bool(sec.get("enabled", False), "pure_torch.enabled")
    kwargs = {k: sec[k] for k in ("use_compile", "use_packing", "target_packed_rows") if k in sec}
    for k in ("use_compile", "use_packing"):
        if k in kwargs and kwargs[k] is not None:
            kwargs[k] = _to_bool(kwargs[k], k)
    if kwargs.get("target_packed_rows") is not None:
        kwargs["target_packed_rows"] = _to_int(kwargs["target_packed_rows"], "target_packed_rows")
    return enabled, PureTorchConfig(**kwargs)


def load_resume_config(section: Optional[Mapping[str, Any]]) -> ResumeConfig:
    if section is None:
        return ResumeConfig(is_resume=False, checkpoint_dir="", extra_epochs=None)
    known = field_names(ResumeConfig)
    extra = sorted(k for k in section if k not in known)
    if extra:
        raise ConfigError(f"Unexpected resume configuration keys: {', '.join(extra)}")
    kwargs = {k: v for k, v in section.items() if v is not None}
    if "is_resume" in kwargs:
        kwargs["is_resume"] = _to_bool(kwargs["is_resume"], "is_resume")
    if kwargs.get("extra_epochs") is not None:
        kwargs["extra_epochs"] = _to_int(kwargs["extra_epochs"], "extra_epochs")
    cfg = ResumeConfig(**kwargs)
    if cfg.is_resume:
        if not cfg.checkpoint_dir:
            raise ConfigError("Resume requested but 'checkpoint_dir' is missing under 'resume'")
        if not Path(cfg.checkpoint_dir).exists():
            raise ConfigError(f"Checkpoint directory does not exist: {cfg.checkpoint_dir}")
    return cfg


def load_student_config(section: Optional[Mapping[str, Any]]) -> StudentConfig:
    if section is None:
        raise ConfigError("Model configuration is required but not found in YAML")
    known = field_names(StudentConfig)
    extra = sorted(k for k in section if k not in known)
    if extra:
        raise ConfigError(f"Unexpected model configuration keys: {', '.join(extra)}")
    kwargs = {k: v for k, v in section.items() if v is not None}
    return StudentConfig(**_coerce(StudentConfig, kwargs))


def load_distill_config(section: Optional[Mapping[str, Any]], require_dataset_dir: bool = True) -> DistillationConfig:
    if section is None:
        raise ConfigError("Distillation configuration is required but not found in YAML")
    cfg = dict(section)
    if require_dataset_dir and not cfg.get("dataset_dir"):
        raise ConfigError("dataset_dir is required in distillation configuration. Run "
                          "'nanoplm data from-yaml' first to prepare the dataset.")
    known = field_names(DistillationConfig)
    extra = sorted(k for k in cfg if k not in known)
    if extra:
        raise ConfigError(f"Unexpected distillation configuration keys: {', '.join(extra)}")
    kwargs = {k: v for k, v in cfg.items() if v is not None}
    if isinstance(kwargs.get("teacher"), Mapping):
        bad = sorted(k for k in kwargs["teacher"] if k not in field_names(TeacherConfig))
        if bad:
            raise ConfigError(f"Unexpected distillation.teacher keys: {', '.join(bad)}")
        kwargs["teacher"] = TeacherConfig(**_coerce(TeacherConfig, dict(kwargs["teacher"])))
    if isinstance(kwargs.get("lr_scheduler_kwargs"), str):
        import json
        kwargs["lr_scheduler_kwargs"] = json.loads(kwargs["lr_scheduler_kwargs"])
    return DistillationConfig(**_coerce(DistillationConfig, kwargs))


def read_yaml(path: str | Path) -> dict:
    import yaml
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"Config file not found: {p}")
    with open(p, "r", encoding="utf-8") as f:
        data = yaml.safe_load(f)
    if not isinstance(data, dict):
        raise ConfigError(f"Config file must contain a mapping at the top level: {p}")
    return data
