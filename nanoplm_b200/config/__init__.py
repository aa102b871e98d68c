from .schema import (DistillationConfig, ModelConfig, MoEConfig, PretrainingConfig, PureTorchConfig,
                     ResumeConfig, StudentConfig, TeacherConfig, as_plain_dict)
from .loaders import (ConfigError, load_distill_config, load_model_config, load_pretrain_config,
                      load_resume_config, load_student_config, read_yaml, resolve_pure_torch_config)
from .datasets import DATASET_URLS

__all__ = [
    "DistillationConfig", "ModelConfig", "MoEConfig", "PretrainingConfig", "PureTorchConfig",
    "ResumeConfig", "StudentConfig", "TeacherConfig", "as_plain_dict", "ConfigError",
    "load_distill_config", "load_model_config", "load_pretrain_config", "load_resume_config",
    "load_student_config", "read_yaml", "resolve_pure_torch_config", "DATASET_URLS",
]
