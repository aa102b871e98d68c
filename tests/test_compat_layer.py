"""`nanoplm_b200.compat`: the reference's import paths and call conventions served by this package
(run in a child process so that the `nanoplm.*` entries never reach this test process's modules)."""
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

SCRIPT = r'''
import sys, torch
import nanoplm_b200.compat as compat
compat.install()
assert compat.installed()
from pathlib import Path
from nanoplm.data.shuffler import FastaShuffler
from nanoplm.data.filterer import Filterer
from nanoplm.data.splitor import Splitor
from nanoplm.data.file_pool import detect_file_limits, ThreadSafeFileHandlePool
from nanoplm.data.manifest import read_manifest, get_dataset_paths
from nanoplm.pretraining.dataset import ShardWriter, ShardedDataset
from nanoplm.pretraining.models.modern_bert import ProtModernBertTokenizer
from nanoplm.pretraining.utils import compute_batch_setup, get_num_workers, prepare_run_and_steps
from nanoplm.pretraining.config import PretrainingConfig, ResumeConfig
from nanoplm.distillation.dataset import SaveKDDataset, LoadKDDataset, KDDatasetOnTheFly, shard_h5_file
from nanoplm.distillation.collator import DistillDataCollator
from nanoplm.distillation.models.teacher import ProtT5, BaseTeacher
from nanoplm.distillation.models.student import ProtX, ProtXConfig, ProtXTokenizer
from nanoplm.utils import create_dirs, get_device, logger, log_stage
from nanoplm.utils.common import read_yaml
from nanoplm_b200.config.schema import TeacherConfig
from nanoplm_b200.data.synthetic import write_synthetic_fasta
from nanoplm_b200.data.fasta import count_fasta

work = Path(sys.argv[1])
log_stage("data")
fasta = write_synthetic_fasta(work / "raw.fasta", 40, 12, 50, seed=5)
# positional order of the reference: (input, output, seed, backend)
FastaShuffler(fasta, work / "shuf.fasta", 7, "biopython").shuffle()
Filterer(work / "shuf.fasta", work / "filt.fasta", 15, 45, -1, 0).filter()
n_train, n_val = Splitor(input_file=work / "filt.fasta", train_file=work / "s" / "tr.fasta",
                         val_file=work / "s" / "va.fasta", val_ratio=0.25).split()
assert n_train == count_fasta(work / "s" / "tr.fasta") and n_val == count_fasta(work / "s" / "va.fasta") and n_val > 0
assert detect_file_limits(num_workers=4, reserve_percentage=0.5) >= 5

tok = ProtModernBertTokenizer(use_bos_token=False)
try:
    ProtModernBertTokenizer(mask_token="[MASK]")
    raise SystemExit("a different mask token must be refused")
except ValueError:
    pass
shards = ShardWriter(fasta_path=str(work / "s" / "tr.fasta"), tokenizer=tok, max_length=64, output_dir=str(work / "sh"),
                     samples_per_shard=10, max_workers=1).create_shards()
assert len(ShardedDataset(data_dir=str(work / "sh"))) == n_train and len(shards) >= 2

cfg = PretrainingConfig(dataset_dir="unused", ckp_dir=str(work / "ck"), global_batch_size=4096, micro_batch_size=8)
bs = compute_batch_setup(cfg, 64, 2)
assert bs.grad_accum_steps == 4 and get_num_workers(0, 1) == 0
name, wb, out, epochs, ls, es, ss, rstep = prepare_run_and_steps(cfg, ResumeConfig(False, "", None), 100, 10)
assert name.startswith("run-") and Path(out).name == name and rstep in (0, None)

small = TeacherConfig(d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4)
teacher = ProtT5(device="cpu", random_init=True, cfg=small)
assert isinstance(teacher, BaseTeacher)
create_dirs(work / "kd" / "x.kdz")
out = SaveKDDataset(work / "s" / "va.fasta", work / "kd" / "val.kdz", teacher, "get_embeddings", 48, 4, "cpu", 1, -1,
                    False).process_dataset()
ds = LoadKDDataset(h5_path=out, device="cpu", seed=1, sharded=False)
assert len(ds) == n_val - 1 and ds[0]["teacher_embeddings"].shape == (48, 32)
parts = shard_h5_file(input_h5_path=out, n_sharded_files=2, output_dir=work / "kd2", total_sequences=len(ds))
assert len(parts) == 2
from nanoplm.data.validation import validate_hdf5_shards, ValidationError
from nanoplm.pretraining.optim import is_muon_optimizer
assert [Path(f).name for f in validate_hdf5_shards(work / "kd2", expected_count=2)] == sorted(Path(f).name for f in parts)
try:
    validate_hdf5_shards(work / "kd2", expected_count=3)
    raise SystemExit("a wrong shard count must be refused")
except ValidationError:
    pass
assert is_muon_optimizer(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=0.1)) is False
feats = [ds[i] for i in range(3)]
batch = DistillDataCollator(on_the_fly=False)(feats)
assert batch["teacher_embeddings"].shape == (3, 48, 32)
raw = list(KDDatasetOnTheFly(input_fasta=work / "s" / "va.fasta", teacher=teacher, max_seq_len=48, device="cpu"))
assert len(raw) == n_val and "raw_sequence" in raw[0]
fly = DistillDataCollator(teacher_model=teacher.encoder_model, teacher_tokenizer=teacher.tokenizer,
                          student_tokenizer=ProtXTokenizer(), on_the_fly=True, max_seq_len=48)(raw[:3])
assert set(fly) == {"input_ids", "attention_mask", "teacher_embeddings"} and fly["teacher_embeddings"].shape == (3, 48, 32)
assert fly["teacher_embeddings"].dtype == torch.float32

student = ProtX(ProtXConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2))
h = student(fly["input_ids"], fly["attention_mask"], training_mode=True)
h = h["last_hidden_state"] if isinstance(h, dict) else h.last_hidden_state
assert h.shape == (3, 48, 1024)
# distillation through the reference's entry point and keyword names
import os
os.environ["WANDB_MODE"] = "disabled"
from nanoplm.distillation.pipeline import DistillationConfig, ResumeConfig as DResume, run_distillation
from nanoplm.data.manifest import DistillationManifest, write_manifest
kd = work / "kd_fly"
write_synthetic_fasta(kd / "train.fasta", 32, 10, 40, seed=1)
write_synthetic_fasta(kd / "val.fasta", 8, 10, 40, seed=2)
write_manifest(kd, DistillationManifest(pipeline_mode="distillation", seqs_num=40, min_seq_len=10, max_seq_len=48,
                                        val_ratio=0.2, train_dir=".", val_dir=".", train_sequences=32, val_sequences=8,
                                        teacher_model="prott5", on_the_fly=True, train_fasta="train.fasta",
                                        val_fasta="val.fasta"))
dcfg = DistillationConfig(dataset_dir=str(kd), ckp_dir=str(work / "dck"), num_epochs=1, batch_size=8, logging_steps=1,
                          eval_steps=2, save_steps=2, bf16=False, teacher_random_init=True,
                          teacher=TeacherConfig(d_model=1024, d_kv=8, d_ff=32, num_layers=1, num_heads=2))
res = run_distillation(model_config=ProtXConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2),
                       distill_config=dcfg, resume_config=DResume(is_resume=False, checkpoint_dir="", extra_epochs=None))
assert res["global_step"] == 4 and (Path(res["output_dir"]) / "checkpoint-4" / "model.safetensors").exists()
(work / "c.yaml").write_text("a: {b: 1}\n")
assert read_yaml(work / "c.yaml") == {"a": {"b": 1}} and get_device() in ("cpu", "cuda")
try:
    from nanoplm.pretraining.collator import NoSuchThing
    raise SystemExit("unknown names must not resolve")
except ImportError:
    pass
compat.uninstall()
assert "nanoplm" not in sys.modules
print("COMPAT OK")
'''


def test_reference_import_paths_and_call_conventions(tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-c", SCRIPT, str(tmp_path)], cwd=tmp_path, env=env, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0 and "COMPAT OK" in out.stdout, (out.stdout + out.stderr)[-4000:]


def test_install_refuses_to_shadow_a_real_package(tmp_path):
    (tmp_path / "nanoplm").mkdir()
    (tmp_path / "nanoplm" / "__init__.py").write_text("REAL = True\n")
    code = ("import nanoplm_b200.compat as c\n"
            "try:\n    c.install()\n    print('installed')\nexcept RuntimeError as e:\n    print('refused')\n"
            "c.install(force=True)\nimport nanoplm\nprint(hasattr(nanoplm, 'REAL'))\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(tmp_path), str(ROOT)]), CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, "-c", code], cwd=tmp_path, env=env, capture_output=True, text=True, timeout=300)
    assert out.stdout.split() == ["refused", "False"], out.stdout + out.stderr
