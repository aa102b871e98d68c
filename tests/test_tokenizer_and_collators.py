"""Tokenizer ids and the behavioural contracts of the MLM / packing collators (the assertions of the
reference's live collator tests, tests/test_packing_collator.py and tests/test_pretraining_collator.py,
plus the static packed format, which the reference leaves untested)."""
import numpy as np
import pytest
import torch

from nanoplm_b200.data.collators import PackingCollator, ProtDataCollatorForLM
from nanoplm_b200.data.packing import pack_ffd, pack_ffd_python
from nanoplm_b200.data.tokenizer import ProtTokenizer, StudentTokenizer, TeacherTokenizer
from nanoplm_b200.models.encoder import position_ids_from_cu_seqlens


@pytest.fixture(scope="module")
def tok():
    return ProtTokenizer()


def _examples(tok, seqs):
    return [{"input_ids": torch.tensor(tok.encode(s)), "attention_mask": torch.ones(len(s) + 1)} for s in seqs]


def test_vocabulary_ids_and_text_handling(tok):
    v = tok.get_vocab()
    assert len(v) == 32 and v["<pad>"] == 0 and v["</s>"] == 1 and v["<unk>"] == 2 and v["<mask>"] == 3
    assert [v[c] for c in "ALGVSREDTIPKFQNYMHWCXBOUZ"] == list(range(4, 29))
    assert v["<s>"] == 29 and v["<unused0>"] == 30 and v["<unused1>"] == 31
    assert tok.encode("MKT") == [20, 15, 12, 1]                      # sequence then </s>
    assert tok.encode("mkt") == tok.encode("MKT")                    # upper-cased
    assert tok.encode("UZOB") == [24, 24, 24, 24, 1]                 # rare residues read as X
    assert tok.encode("M*") == [20, 2, 1]                            # unknown character
    assert ProtTokenizer(use_bos_token=True).encode("MK") == [29, 20, 15, 1]
    assert tok.encode("MKTAY", max_length=3) == [20, 15, 1]             # truncation keeps </s> (as the reference does)
    assert tok.all_special_ids == [0, 1, 2, 3]
    assert tok.decode([20, 15, 12, 1], skip_special_tokens=True) == "MKT"


def test_student_and_teacher_tokenizers():
    s = StudentTokenizer()
    assert s.vocab_size == 28 and s.mask_token_id is None
    assert s.encode("AL") == [3, 4, 1] and s.encode("a") == [2, 1]   # no normalisation: lower case -> unk
    t = TeacherTokenizer()
    assert t.vocab_size == 128
    assert TeacherTokenizer.preprocess(" mkUz ") == "M K X X"
    assert t.encode(TeacherTokenizer.preprocess("MKU")) == t.encode("MKX")


def test_padding_collator_shapes_and_labels(tok):
    c = ProtDataCollatorForLM(tok, mlm_probability=0.3, seed=0)
    b = c(_examples(tok, ["MKTAYIAKQR", "MK", "ACDEFGHIK"]))
    assert b["input_ids"].shape == (3, 11) and b["input_ids"].dtype == torch.long
    assert b["attention_mask"].sum(1).tolist() == [11, 3, 10]
    lab, ids = b["labels"], b["input_ids"]
    assert ((lab == -100) | (lab >= 4)).all()                        # only residues are ever targets
    assert (lab[b["attention_mask"] == 0] == -100).all()
    untouched = lab == -100
    orig = tok.pad(_examples(tok, ["MKTAYIAKQR", "MK", "ACDEFGHIK"]))["input_ids"]
    assert (ids[untouched] == orig[untouched]).all()


def test_special_tokens_are_never_masked_even_at_probability_one(tok):
    c = ProtDataCollatorForLM(tok, mlm_probability=1.0, seed=1)
    b = c(_examples(tok, ["MKTAYIAKQR", "MKT"]))
    eos_pos = b["attention_mask"].sum(1) - 1
    for r, p in enumerate(eos_pos.tolist()):
        assert b["labels"][r, p] == -100 and b["input_ids"][r, p] == 1
    assert (b["labels"][b["attention_mask"] == 1] != -100).sum() == 10 + 3


def test_mask_random_keep_split_follows_the_normalised_proportions(tok):
    c = ProtDataCollatorForLM(tok, 1.0, mask_token_probability=8, random_token_probability=1, keep_probability=1, seed=2)
    assert abs(c.p_mask - 0.8) < 1e-9 and abs(c.p_rand - 0.1) < 1e-9 and abs(c.p_keep - 0.1) < 1e-9
    seq = "ACDEFGHIKLMNPQRSTVWY" * 20
    n_mask = n_keep = n_rand = 0
    for _ in range(20):
        b = c(_examples(tok, [seq]))
        ids, lab = b["input_ids"][0, :-1], b["labels"][0, :-1]
        n_mask += int((ids == 3).sum())
        n_keep += int((ids == lab).sum())
        n_rand += int(((ids != 3) & (ids != lab)).sum())
        assert (ids >= 3).all()                                      # replacements never are pad/eos/unk
    tot = n_mask + n_keep + n_rand
    assert abs(n_mask / tot - 0.8) < 0.03
    assert 0.07 < (n_rand / tot) < 0.13                              # some random draws equal the original
    assert set(c.allowed_random_token_ids.tolist()) == set(range(4, 32))


def test_empty_batch_and_missing_mask_token():
    class NoMask(StudentTokenizer):
        pass
    with pytest.raises(ValueError):
        ProtDataCollatorForLM(NoMask())


def test_ffd_packer_matches_the_python_reference():
    rng = np.random.default_rng(0)
    for n, w in ((1, 16), (50, 64), (300, 512)):
        lens = rng.integers(1, w + 20, size=n)
        o, r, s, nr = pack_ffd(lens, w)
        o2, r2, nr2 = pack_ffd_python(lens.tolist(), w)
        assert nr == nr2 and o.tolist() == o2 and r.tolist() == r2
        fill = np.zeros(nr, dtype=int)
        for k in range(n):
            assert s[k] == fill[r[k]]
            fill[r[k]] += min(int(lens[o[k]]), w)
        assert (fill <= w).all()


def test_dynamic_packing_structure(tok):
    seqs = ["MKTAYIAKQR" * 3, "MK", "ACDEFGHIK", "MKTAYIAKQRQISFVKSHFSRQ", "A" * 70]
    c = PackingCollator(tok, max_seq_len=64, mlm_probability=0.3, seed=3)
    b = c(_examples(tok, seqs))
    R, W = b["input_ids"].shape
    assert W == 64 and R < len(seqs)                                 # rows are shared
    cu = b["cu_seqlens"]
    assert cu.dtype == torch.int32 and cu[0] == 0 and len(cu) == len(seqs) + 1
    lens = (cu[1:] - cu[:-1]).tolist()
    assert sorted(lens) == sorted(min(len(s) + 1, 64) for s in seqs)  # no token lost, long ones truncated
    assert b["max_seqlen"] == max(lens) and int(b["attention_mask"].sum()) == int(cu[-1])
    assert int(b["attention_mask"].sum()) / (R * W) > 0.5
    pos = position_ids_from_cu_seqlens(cu, int(cu[-1]))
    for a, e in zip(cu[:-1].tolist(), cu[1:].tolist()):
        assert pos[a:e].tolist() == list(range(e - a))
    assert (b["labels"][b["attention_mask"] == 0] == -100).all()
    assert (b["input_ids"][b["attention_mask"] == 0] == 0).all()


def test_static_packing_format(tok):
    seqs = ["MKTAYIAKQR" * 2, "MK", "ACDEFGHIK", "MKTAYIAKQRQISFVKSHFSRQ"]
    c = PackingCollator(tok, max_seq_len=32, mlm_probability=0.5, target_rows=4, batch_size=4, seed=4)
    b = c(_examples(tok, seqs))
    F = 4 * 32
    assert b["input_ids"].shape == (F,) and b["labels"].shape == (F,) and b["position_ids"].shape == (F,)
    assert b["position_ids"].dtype == torch.int32 and b["max_seqlen"] == 32
    cu = b["cu_seqlens"]
    assert len(cu) == 4 + 1 + 4 and cu[-1] == F and (cu[1:] >= cu[:-1]).all()
    T = int(cu[4])
    assert T == sum(len(s) + 1 for s in seqs) == b["num_real_tokens"]
    assert (cu[5:] - cu[4:-1]).max() <= 32                           # the padding tail is cut into chunks <= W
    assert (b["input_ids"][T:] == 0).all() and (b["labels"][T:] == -100).all()
    idx = b["masked_idx"].long()
    assert (b["labels"][idx] == b["masked_labels"].long()).all() and (b["labels"] != -100).sum() == len(idx)


def test_static_packing_drops_whole_rows_instead_of_failing(tok):
    seqs = ["A" * 30] * 8
    c = PackingCollator(tok, max_seq_len=32, mlm_probability=0.3, target_rows=4, batch_size=8, seed=5)
    b = c(_examples(tok, seqs))
    assert b["num_real_tokens"] == 4 * 31 and c.dropped_sequences == 4
    assert b["input_ids"].shape == (128,)


def test_balanced_batch_sampler_deals_equal_cost_bins_and_resumes():
    """Every rank's micro-batches of an optimizer step cost the same, the step's global batch is the
    shuffled sampler's window, ranks never share a sequence, and fast_forward resumes mid-epoch."""
    import numpy as np
    from nanoplm_b200.data.packing import balance_bins, balance_bins_python
    from nanoplm_b200.data.sampler import BalancedBatchSampler
    rng = np.random.default_rng(3)
    lens = rng.integers(20, 513, size=4 * 2 * 26 * 5 + 17).astype(np.int32)    # 5 whole steps + a remainder
    b, c = balance_bins(lens[:208], 8, 26)
    b2, c2 = balance_bins_python(lens[:208].tolist(), 8, 26)
    assert b.tolist() == b2 and np.allclose(c, c2)
    world, accum, mbs = 4, 2, 26
    samplers = [BalancedBatchSampler(lens, mbs, accum, world, r, True, seed=7) for r in range(world)]
    batches = [list(s) for s in samplers]
    assert all(len(bt) == 5 * accum == len(samplers[0]) for bt in batches)
    cost = lens + lens.astype(np.float64) ** 2 / 2700.0
    for step in range(5):
        per_rank = [sum(cost[i] for a in range(accum) for i in batches[r][step * accum + a]) for r in range(world)]
        assert max(per_rank) / (sum(per_rank) / world) < 1.002
        seen = [i for r in range(world) for a in range(accum) for i in batches[r][step * accum + a]]
        assert len(seen) == len(set(seen)) == world * accum * mbs
        g = torch.Generator()
        g.manual_seed(7)
        window = torch.randperm(len(lens), generator=g)[step * len(seen):(step + 1) * len(seen)].tolist()
        assert sorted(seen) == sorted(window)
        assert all(len(batches[r][step * accum + a]) == mbs for r in range(world) for a in range(accum))
    s = samplers[1]
    s.fast_forward(3)
    assert len(s) == 5 * accum - 3 and list(s) == batches[1][3:]
    assert list(s) == batches[1]                   # the offset applies to one epoch only
    s.set_epoch(1)
    assert list(s) != batches[1]
