"""Utilities around the distillation models that have a reference counterpart but no place in the
training loop: embedding generation from a saved student and checkpoint inspection
(student/model.py:111-497), the `ProtT5` / `BaseTeacher` interface (teacher/base.py, teacher/prott5.py),
the on-the-fly FASTA dataset (distillation/dataset.py:21-52) and the dataset URL table
(config/datasets.py:13-24)."""
import pytest
import torch

from nanoplm_b200.config.schema import StudentConfig, TeacherConfig


def _student():
    from nanoplm_b200.models.student import ProtX
    torch.manual_seed(0)
    m = ProtX(StudentConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=2))
    with torch.no_grad():                                   # the output projections start at zero
        for n, p in m.named_parameters():
            if n.endswith("Wo.weight"):
                p.normal_(0, 0.05)
    return m.float().eval()


def test_saved_student_embeds_sequences_and_reports_its_architecture(tmp_path):
    from safetensors.torch import save_file

    from nanoplm_b200.models.student import (calculate_model_parameters, inspect_checkpoint_architecture,
                                             load_and_generate_embeddings, print_parameter_breakdown)
    m = _student()
    save_file({k: v.contiguous() for k, v in m.state_dict().items()}, str(tmp_path / "model.safetensors"))
    torch.save(m.state_dict(), tmp_path / "pytorch_model.bin")
    info = inspect_checkpoint_architecture(tmp_path / "model.safetensors")
    assert info["hidden_size"] == 64 and info["num_hidden_layers"] == 3 and info["intermediate_size"] == 128
    assert info["projection_layer"] is True and info["vocab_size"] == 28
    counts = calculate_model_parameters(m)
    assert counts["total"] == info["num_parameters"] == sum(p.numel() for p in m.parameters())
    assert counts["trainable"] == counts["total"] and counts["frozen"] == 0
    groups = print_parameter_breakdown(m)
    assert groups["total"] == counts["total"] and groups["projection"] == 64 * 1024
    assert groups["attention"] > 0 and groups["mlp"] > 0 and groups["other"] == 0

    seqs = ["MKTAYIAKQRQISFVK", "ACDEFG", "MKV"]
    cfg = StudentConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=2)
    pooled = load_and_generate_embeddings(tmp_path, seqs, cfg, batch_size=2, device=torch.device("cpu"))
    per_tok = load_and_generate_embeddings(tmp_path / "pytorch_model.bin", seqs, cfg, per_token=True,
                                           device=torch.device("cpu"))
    assert [tuple(p.shape) for p in pooled] == [(64,)] * 3
    assert [tuple(p.shape) for p in per_tok] == [(16, 64), (6, 64), (3, 64)]    # one row per residue, no </s>
    for a, b in zip(pooled, per_tok):
        assert torch.allclose(a, b.mean(0), atol=1e-5)
    # a sequence embeds the same alone and inside a padded batch
    alone = load_and_generate_embeddings(tmp_path, [seqs[2]], cfg, device=torch.device("cpu"))[0]
    assert torch.allclose(alone, pooled[2], atol=1e-4)
    # without a config the geometry comes from the file (heads = hidden / 64)
    guessed = load_and_generate_embeddings(tmp_path, seqs[:1], device=torch.device("cpu"))
    assert tuple(guessed[0].shape) == (64,)
    with pytest.raises(KeyError):
        bad = dict(m.state_dict(), extra=torch.zeros(1))
        torch.save(bad, tmp_path / "bad.bin")
        load_and_generate_embeddings(tmp_path / "bad.bin", seqs[:1], cfg, device=torch.device("cpu"))


def test_prott5_wrapper_has_the_reference_teacher_interface(tmp_path):
    from nanoplm_b200.data.kd_dataset import LoadKDDataset, SaveKDDataset
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    from nanoplm_b200.models.teacher import BaseTeacher, ProtT5, T5EncoderTeacher
    small = TeacherConfig(d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4)
    t = ProtT5(device="cpu", random_init=True, cfg=small, seed=3)
    assert isinstance(t, BaseTeacher) and t.model_name == "Rostlab/prot_t5_xl_uniref50"
    assert t.preprocess(" mkUzob ") == "M K X X X X" and t.preprocess(None) == ""
    assert isinstance(t.encoder_model, T5EncoderTeacher) and t.encoder_model is t.encoder_model     # cached
    assert not any(p.requires_grad for p in t.encoder_model.parameters())
    h, mask = t.embed(["MKTAYIAK", "MK"])
    assert h.shape == (2, 9, 32) and mask.sum(1).tolist() == [9, 3]
    padded, _ = t.embed(["MKTAYIAK", "MK"], max_length=16)
    assert torch.allclose(padded[1, :3], h[1, :3], atol=1e-5)
    assert t.get_layer_by_name("shared.weight").shape == (128, 32)
    with pytest.raises(ValueError):
        t.get_layer_by_name("nope")
    with pytest.raises(NotImplementedError):
        BaseTeacher("cpu").preprocess("A")
    # the wrapper is accepted where a teacher module is
    fasta = write_synthetic_fasta(tmp_path / "a.fasta", 5, 8, 20, seed=3)
    files = SaveKDDataset(fasta, tmp_path / "kd.kdz", max_seq_len=24, batch_size=4, device="cpu",
                          samples_per_shard=-1, teacher=t).run()
    assert LoadKDDataset(files[0])[0]["teacher_embeddings"].shape == (24, 32)


def test_on_the_fly_dataset_splits_the_fasta_over_ranks_and_workers(tmp_path):
    from torch.utils.data import DataLoader

    from nanoplm_b200.data.fasta import iter_fasta
    from nanoplm_b200.data.kd_dataset import KDDatasetOnTheFly
    from nanoplm_b200.data.synthetic import write_synthetic_fasta
    fasta = write_synthetic_fasta(tmp_path / "a.fasta", 23, 8, 20, seed=1)
    all_seqs = [s for _, s in iter_fasta(fasta)]
    assert [d["raw_sequence"] for d in KDDatasetOnTheFly(fasta)] == all_seqs
    assert [d["raw_sequence"] for d in KDDatasetOnTheFly(fasta, max_seqs_num=7)] == all_seqs[:7]
    parts = [[d["raw_sequence"] for d in KDDatasetOnTheFly(fasta, rank=r, world=3)] for r in range(3)]
    assert sorted(sum(parts, [])) == sorted(all_seqs) and max(map(len, parts)) - min(map(len, parts)) <= 1
    # two ranks with two loader workers each: four disjoint strides that cover the file once
    got = []
    for r in range(2):
        loader = DataLoader(KDDatasetOnTheFly(fasta, rank=r, world=2), batch_size=None, num_workers=2)
        mine = [d["raw_sequence"] for d in loader]
        assert 11 <= len(mine) <= 12
        got += mine
    assert sorted(got) == sorted(all_seqs)
    with pytest.raises(FileNotFoundError):
        KDDatasetOnTheFly(tmp_path / "missing.fasta")


def test_dataset_url_table_matches_the_reference_keys():
    from nanoplm_b200.config.datasets import DATASET_URLS, get_supported_datasets, resolve_dataset_url
    assert set(DATASET_URLS) == {"swissprot", "trembl", "uniref50", "uniref90", "uniref100"}
    assert all(u.startswith("https://ftp.uniprot.org/pub/databases/uniprot/") and u.endswith(".fasta.gz")
               for u in DATASET_URLS.values())
    assert get_supported_datasets() == DATASET_URLS and get_supported_datasets() is not DATASET_URLS
    assert resolve_dataset_url("UniRef50", None).endswith("uniref50.fasta.gz")
    assert resolve_dataset_url("anything", "http://x/y.gz") == "http://x/y.gz"
    with pytest.raises(KeyError):
        resolve_dataset_url("pfam", None)
    with pytest.raises(KeyError):
        resolve_dataset_url(None, None)


def test_compat_student_utilities_follow_the_reference_call_convention(tmp_path):
    """`nanoplm.distillation.models.student.ProtX.<utility>` as served by `nanoplm_b200.compat`: static
    methods taking (embed_dim, num_layers, num_heads, ...) or a checkpoint path, the embedding
    generator yielding (sequence, tensor) pairs (student/model.py:111-497)."""
    from safetensors.torch import save_file

    from nanoplm_b200.compat.adapters import ProtX
    m = _student()
    save_file({k: v.contiguous() for k, v in m.state_dict().items()}, str(tmp_path / "model.safetensors"))
    assert ProtX.inspect_checkpoint_architecture(str(tmp_path / "model.safetensors")) == (64, 3, 1)
    with pytest.raises(FileNotFoundError):
        ProtX.inspect_checkpoint_architecture(str(tmp_path / "missing.safetensors"))
    n = ProtX.calculate_model_parameters(64, 3, 2)
    assert n == sum(p.numel() for p in ProtX(StudentConfig(hidden_size=64, intermediate_size=256, num_hidden_layers=3,
                                                           num_attention_heads=2)).parameters())
    assert ProtX.calculate_model_parameters(64, 3, 2, projection_layer=False) == n - 64 * 1024 - 1024
    ProtX.print_parameter_breakdown(64, 3, 2)
    seqs = ["MKTAYIAKQRQISFVK", "ACDEFG"]
    pooled = list(ProtX.load_and_generate_embeddings(str(tmp_path / "model.safetensors"), iter(seqs), batch_size=2,
                                                     device="cpu"))
    assert [s for s, _ in pooled] == seqs and all(tuple(e.shape) == (64,) for _, e in pooled)
    per_tok = list(ProtX.load_and_generate_embeddings(str(tmp_path / "model.safetensors"), seqs, device="cpu",
                                                      per_seq_embeddings=False, max_length=5))
    assert [tuple(e.shape) for _, e in per_tok] == [(4, 64), (4, 64)]          # truncated to max_length - 1 residues
