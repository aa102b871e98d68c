from .tokenizer import ProtTokenizer, StudentTokenizer, TeacherTokenizer
from .manifest import (MANIFEST_FILENAME, DistillationManifest, PretrainManifest, read_manifest,
                       validate_manifest_for_pipeline, write_manifest, get_dataset_paths)

__all__ = [
    "ProtTokenizer", "StudentTokenizer", "TeacherTokenizer", "MANIFEST_FILENAME",
    "DistillationManifest", "PretrainManifest", "read_manifest", "validate_manifest_for_pipeline",
    "write_manifest", "get_dataset_paths",
]
