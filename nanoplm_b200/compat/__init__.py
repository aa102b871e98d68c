"""Import paths of the reference package, served by this one.

Code written against `nanoplm` (`from nanoplm.pretraining.collator import PackingCollator`,
`from nanoplm.pretraining.pure_pipeline import run_pure_pretraining`, ...) keeps working after

    import nanoplm_b200.compat
    nanoplm_b200.compat.install()

which registers module objects under the reference's dotted names (`MODULES` below lists every module
and name) whose attributes resolve, on first use, to this package's classes and functions, through
`compat/adapters.py` where the call convention differs. Nothing is installed when a real `nanoplm`
package is importable, unless `force=True`. `python -m pytest -p nanoplm_b200.compat.pytest_plugin` does
the same before test collection (that is how the reference's own unit tests are run against this
package in `tests/test_reference_own_tests.py`).
"""
from __future__ import annotations

import importlib
import importlib.util
import sys
import types

A = "nanoplm_b200.compat.adapters"

# reference module -> {name there: "module here[:attribute]"}
MODULES: dict[str, dict[str, str]] = {
    "nanoplm": {"__version__": "nanoplm_b200:__version__"},
    "nanoplm.cli": {"cli": "nanoplm_b200.cli", "main": "nanoplm_b200.cli"},
    "nanoplm.cli.data": {"data": "nanoplm_b200.cli.data"},
    "nanoplm.cli.pretrain": {"pretrain": "nanoplm_b200.cli.pretrain"},
    "nanoplm.cli.distill": {"distill": "nanoplm_b200.cli.distill"},
    "nanoplm.config": {},
    "nanoplm.config.datasets": {"DATASET_URLS": "nanoplm_b200.config.datasets",
                                "get_supported_datasets": "nanoplm_b200.config.datasets"},
    "nanoplm.utils": {"logger": "nanoplm_b200.utils.logging", "log_stage": A, "create_dirs": A, "get_device": A,
                      "get_caller_dir": A},
    "nanoplm.utils.logger": {"logger": "nanoplm_b200.utils.logging", "log_stage": A},
    "nanoplm.utils.common": {"read_yaml": A, "create_dirs": A, "get_device": A, "get_caller_dir": A,
                             "is_flash_attention_available": A, "inside_git_repo": A, "is_git_subdir": A,
                             "resolve_world_size": "nanoplm_b200.runtime.run_dirs"},
    "nanoplm.data": {},
    "nanoplm.data.downloader": {"Downloader": "nanoplm_b200.data.prep", "DownloadError": "nanoplm_b200.data.prep"},
    "nanoplm.data.extractor": {"Extractor": "nanoplm_b200.data.prep", "ExtractionError": "nanoplm_b200.data.prep"},
    "nanoplm.data.shuffler": {"FastaShuffler": A, "ShufflingError": "nanoplm_b200.data.prep"},
    "nanoplm.data.filterer": {"Filterer": "nanoplm_b200.data.prep", "FilterError": "nanoplm_b200.data.prep"},
    "nanoplm.data.splitor": {"Splitor": A, "SplitError": "nanoplm_b200.data.prep"},
    "nanoplm.data.manifest": {n: "nanoplm_b200.data.manifest" for n in (
        "DataManifestBase", "PretrainManifest", "DistillationManifest", "write_manifest", "read_manifest",
        "validate_manifest_for_pipeline", "get_dataset_paths")},
    "nanoplm.data.validation": {**{n: "nanoplm_b200.data.validation" for n in (
        "ValidationError", "validate_pretrain_shards", "validate_pretrain_dataset", "validate_distillation_dataset")},
        "validate_hdf5_shards": A},
    "nanoplm.data.file_pool": {"ThreadSafeFileHandlePool": "nanoplm_b200.data.file_pool", "detect_file_limits": A},
    "nanoplm.pretraining": {"run_pretraining": "nanoplm_b200.runtime.pretrain",
                            "run_pure_pretraining": "nanoplm_b200.runtime.pretrain",
                            "BatchSetup": "nanoplm_b200.runtime.run_dirs", "compute_batch_setup": A},
    "nanoplm.pretraining.config": {n: "nanoplm_b200.config.schema" for n in (
        "PretrainingConfig", "ResumeConfig", "PureTorchConfig")},
    "nanoplm.pretraining.pipeline": {"run_pretraining": "nanoplm_b200.runtime.pretrain",
                                     "PretrainingConfig": "nanoplm_b200.config.schema",
                                     "ResumeConfig": "nanoplm_b200.config.schema"},
    "nanoplm.pretraining.pure_pipeline": {"run_pure_pretraining": "nanoplm_b200.runtime.pretrain"},
    "nanoplm.pretraining.dataset": {n: "nanoplm_b200.data.shards" for n in (
        "ShardWriter", "ShardedDataset", "LazyFastaDataset")},
    "nanoplm.pretraining.collator": {"PackingCollator": "nanoplm_b200.data.collators",
                                     "ProtDataCollatorForLM": "nanoplm_b200.data.collators"},
    "nanoplm.pretraining.utils": {"BatchSetup": "nanoplm_b200.runtime.run_dirs", "compute_batch_setup": A,
                                  "get_num_workers": "nanoplm_b200.runtime.run_dirs", "prepare_run_and_steps": A},
    "nanoplm.pretraining.optim": {"is_muon_optimizer": A},
    "nanoplm.pretraining.models": {},
    "nanoplm.pretraining.models.modern_bert": {"ProtModernBertTokenizer": A, "PureProtModernBertMLM": A,
                                               "ProtModernBertMLM": A + ":PureProtModernBertMLM"},
    "nanoplm.pretraining.models.modern_bert.tokenizer": {"ProtModernBertTokenizer": A},
    "nanoplm.pretraining.models.modern_bert.model": {
        "ProtModernBertMLMConfig": "nanoplm_b200.config.schema:ModelConfig",
        "ProtModernBertMLM": A + ":PureProtModernBertMLM"},
    "nanoplm.pretraining.models.modern_bert.pure_model": {"PureProtModernBertMLM": A},
    "nanoplm.pretraining.models.modern_bert.modeling": {
        "_position_ids_from_cu_seqlens": "nanoplm_b200.models.encoder:position_ids_from_cu_seqlens",
        "ModernBertForMaskedLM": "nanoplm_b200.models.encoder:ProtEncoderMLM",
        "ModernBertConfig": "nanoplm_b200.config.schema:ModelConfig"},
    "nanoplm.distillation": {},
    "nanoplm.distillation.pipeline": {"DistillationConfig": "nanoplm_b200.config.schema",
                                      "ResumeConfig": "nanoplm_b200.config.schema", "run_distillation": A},
    "nanoplm.distillation.collator": {"DistillDataCollator": A},
    "nanoplm.distillation.dataset": {n: A for n in ("KDDatasetOnTheFly", "SaveKDDataset", "LoadKDDataset",
                                                     "shard_h5_file")},
    "nanoplm.distillation.models": {},
    "nanoplm.distillation.models.student": {"ProtX": A, "ProtXTokenizer": A,
                                            "ProtXConfig": "nanoplm_b200.config.schema:StudentConfig"},
    "nanoplm.distillation.models.student.model": {"ProtX": A,
                                                  "ProtXConfig": "nanoplm_b200.config.schema:StudentConfig"},
    "nanoplm.distillation.models.student.tokenizer": {"ProtXTokenizer": A},
    "nanoplm.distillation.models.teacher": {"BaseTeacher": "nanoplm_b200.models.teacher",
                                            "ProtT5": "nanoplm_b200.models.teacher"},
    "nanoplm.distillation.models.teacher.base": {"BaseTeacher": "nanoplm_b200.models.teacher"},
    "nanoplm.distillation.models.teacher.prott5": {"ProtT5": "nanoplm_b200.models.teacher"},
}


def _make(name: str, table: dict[str, str]) -> types.ModuleType:
    mod = types.ModuleType(name, f"`{name}` served by nanoplm_b200 (see nanoplm_b200.compat)")
    mod.__path__ = []                                  # a package: sub-modules are looked up in sys.modules
    mod.__all__ = sorted(table)

    def resolve(attr: str):
        target = table.get(attr)
        if target is None:
            raise AttributeError(f"module {name!r} has no attribute {attr!r} (not provided by nanoplm_b200.compat)")
        where, _, what = target.partition(":")
        value = getattr(importlib.import_module(where), what or attr)
        setattr(mod, attr, value)
        return value

    mod.__getattr__ = resolve
    return mod


def installed() -> bool:
    return getattr(sys.modules.get("nanoplm"), "__nanoplm_b200_compat__", False)


def install(force: bool = False) -> None:
    """Registers the `nanoplm.*` names. A real `nanoplm` installation is left alone unless forced."""
    if installed():
        return
    if not force:
        real = "nanoplm" in sys.modules
        try:
            real = real or importlib.util.find_spec("nanoplm") is not None
        except (ImportError, ValueError):
            pass
        if real:
            raise RuntimeError("a `nanoplm` package is importable here; call install(force=True) to shadow it")
    for name in list(sys.modules):
        if name == "nanoplm" or name.startswith("nanoplm."):
            del sys.modules[name]
    for name, table in MODULES.items():
        sys.modules[name] = _make(name, table)
    for name in MODULES:                                # parents expose their sub-modules as attributes
        parent, _, child = name.rpartition(".")
        if parent:
            setattr(sys.modules[parent], child, sys.modules[name])
    sys.modules["nanoplm"].__nanoplm_b200_compat__ = True


def uninstall() -> None:
    if installed():
        for name in list(sys.modules):
            if name == "nanoplm" or name.startswith("nanoplm."):
                del sys.modules[name]
