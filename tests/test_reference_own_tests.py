"""The reference's own live unit tests, run unmodified against this package.

`tests/test_packing_collator.py` and `tests/test_pretraining_collator.py` of the reference checkout are
its two test files that still import there; `tests/test_fasta_dataset.py` no longer does, because it
names a `LazyFastaDataset` the reference dropped, but its tests describe the shard writer, the sharded
dataset and that lazy dataset, all of which exist here. The files import
`nanoplm.pretraining.{collator, dataset}`, `...modern_bert.tokenizer` and `...modern_bert.modeling`; here
those module paths are served by `nanoplm_b200.compat` (its pytest plugin registers them before
collection), and pytest runs the reference's files as they are, in a child process. Skipped when no reference checkout is found (`NANOPLM_REFERENCE_DIR`, default: a
`reference` directory beside the repository)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = Path(os.environ.get("NANOPLM_REFERENCE_DIR", ROOT.parent / "reference"))
FILES = ["test_packing_collator.py", "test_pretraining_collator.py", "test_fasta_dataset.py"]

@pytest.mark.skipif(not all((REF_DIR / "tests" / f).exists() for f in FILES), reason="no reference checkout")
def test_reference_unit_tests_pass_on_this_package(tmp_path):
    (tmp_path / "empty.ini").write_text("[pytest]\n")
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    # no conftest, no ini file and importlib import mode: nothing of the reference's source tree gets on
    # sys.path; the plugin registers the `nanoplm.*` names before the test modules are imported
    cmd = [sys.executable, "-m", "pytest", *[str(REF_DIR / "tests" / f) for f in FILES], "--noconftest",
           "-p", "no:cacheprovider", "-p", "nanoplm_b200.compat.pytest_plugin", "-c", str(tmp_path / "empty.ini"),
           "--rootdir", str(tmp_path), "--import-mode=importlib", "-q", "-rA"]
    out = subprocess.run(cmd, cwd=tmp_path, env=env, capture_output=True, text=True, timeout=900)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-4000:]
    assert "34 passed" in text and "failed" not in text.split("short test summary info")[-1], text[-2000:]
    # the classes under test came from this package, not from the reference
    probe = subprocess.run([sys.executable, "-c", "import nanoplm_b200.compat as k; k.install(force=True); "
                            "import nanoplm.pretraining.collator as c; "
                            "print(c.PackingCollator.__module__, c.ProtDataCollatorForLM.__module__)"],
                           cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert probe.stdout.split() == ["nanoplm_b200.data.collators", "nanoplm_b200.data.collators"], probe.stderr[-2000:]


@pytest.mark.skipif(not (REF_DIR / "README.md").exists(), reason="no reference checkout")
def test_yaml_examples_of_the_reference_readme_load_here():
    """The three YAML files printed in the reference's README (params.yaml, pretrain.yaml, distill.yaml;
    README.md:91-333, whose values differ from the `get-yaml` templates) pass this package's strict
    loaders unchanged."""
    import re

    import yaml

    from nanoplm_b200.config import loaders
    blocks = [yaml.safe_load(b) for b in re.findall(r"```ya?ml\n(.*?)```", (REF_DIR / "README.md").read_text(), flags=re.S)]
    blocks = [b for b in blocks if isinstance(b, dict)]
    kinds = set()
    for doc in blocks:
        if "pretraining" in doc:
            model = loaders.load_model_config(doc["model"])
            cfg = loaders.load_pretrain_config(doc["pretraining"])
            enabled, pure = loaders.resolve_pure_torch_config(doc)
            loaders.load_resume_config(doc.get("resume"))
            assert model.hidden_size > 0 and cfg.global_batch_size > 0 and isinstance(enabled, bool) and pure is not None
            kinds.add("pretrain")
        elif "distillation" in doc:
            student = loaders.load_student_config(doc["model"])
            cfg = loaders.load_distill_config(doc["distillation"])
            loaders.load_resume_config(doc.get("resume"))
            assert student.projection_layer in (True, False) and cfg.batch_size > 0
            kinds.add("distill")
        elif "data_params" in doc:
            assert {"pretrain_config", "distillation_config", "data_dirs"} <= set(doc)
            assert doc["data_params"]["pipeline_mode"] in ("none", "pretrain", "distillation")
            kinds.add("data")
    assert kinds == {"pretrain", "distill", "data"}
