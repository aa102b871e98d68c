"""Property tests (hypothesis) for the host-side building blocks that every batch goes through: the
C++ packer and rank balancer against their plain-Python restatements, the packing collator's
invariants for arbitrary sequence sets, the tokenizers, and the balanced sampler's partition."""
import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from nanoplm_b200.data.collators import PackingCollator
from nanoplm_b200.data.packing import balance_bins, balance_bins_python, pack_ffd, pack_ffd_python
from nanoplm_b200.data.sampler import BalancedBatchSampler
from nanoplm_b200.data.tokenizer import ProtTokenizer, StudentTokenizer
from nanoplm_b200.models.encoder import position_ids_from_cu_seqlens

LETTERS = "ALGVSREDTIPKFQNYMHWCXBOUZ"


@settings(max_examples=60, deadline=None, derandomize=True)
@given(st.lists(st.integers(1, 700), min_size=1, max_size=120), st.sampled_from([16, 64, 512]))
def test_packer_matches_python_and_never_overfills(lengths, width):
    order, row_of, start_of, n_rows = pack_ffd(np.asarray(lengths), width)
    o2, r2, n2 = pack_ffd_python(lengths, width)
    assert n_rows == n2 and order.tolist() == list(o2) and row_of.tolist() == list(r2)
    # entry k of the three arrays describes sequence order[k]: its row and its first column there
    assert sorted(order.tolist()) == list(range(len(lengths)))
    fill = np.zeros(n_rows, dtype=np.int64)
    for k, i in enumerate(order.tolist()):
        n = min(lengths[i], width)
        assert 0 <= row_of[k] < n_rows and start_of[k] == fill[row_of[k]] and start_of[k] + n <= width
        fill[row_of[k]] += n
    assert fill.max() <= width and fill.min() > 0
    assert n_rows >= -(-int(np.minimum(lengths, width).sum()) // width)          # never below the volume bound


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.integers(1, 6), st.integers(1, 9), st.data())
def test_rank_balancer_matches_python_and_fills_every_bin(n_bins, per_bin, data):
    lengths = data.draw(st.lists(st.integers(1, 1024), min_size=n_bins * per_bin, max_size=n_bins * per_bin))
    bin_of, cost = balance_bins(np.asarray(lengths), n_bins, per_bin)
    b2, c2 = balance_bins_python(lengths, n_bins, per_bin)
    assert bin_of.tolist() == list(b2) and np.allclose(cost, c2)
    assert np.bincount(bin_of, minlength=n_bins).tolist() == [per_bin] * n_bins


@settings(max_examples=40, deadline=None, derandomize=True)
@given(st.lists(st.text(alphabet=LETTERS, min_size=1, max_size=90), min_size=1, max_size=24), st.booleans(),
       st.integers(0, 2 ** 31 - 1))
def test_packing_collator_keeps_every_token_and_masks_only_residues(seqs, static, seed):
    tok = ProtTokenizer()
    ex = [{"input_ids": torch.tensor(tok.encode(s))} for s in seqs]
    kw = dict(target_rows=len(seqs), batch_size=len(seqs)) if static else {}
    clean = PackingCollator(tok, 64, 0.0, seed=seed, **kw)(ex)
    out = PackingCollator(tok, 64, 0.3, seed=seed, **kw)(ex)
    cu = clean["cu_seqlens"].long()
    lens_in = sorted(min(len(e["input_ids"]), 64) for e in ex)
    real = (cu[1:] - cu[:-1])[: len(seqs)] if static else (cu[1:] - cu[:-1])
    assert sorted(real.tolist()) == lens_in and int(clean["max_seqlen"]) <= 64
    ids, lab = out["input_ids"].reshape(-1), out["labels"].reshape(-1)
    base = clean["input_ids"].reshape(-1)
    assert torch.equal(clean["cu_seqlens"], out["cu_seqlens"])
    m = lab != -100
    assert torch.equal(lab[m], base[m]) and torch.equal(ids[~m], base[~m])
    assert bool((base[m] >= 4).all())                                            # pad / eos / unk / mask never selected
    if static:
        pos = clean["position_ids"]
        total = int(cu[len(seqs)])
        assert torch.equal(pos[:total], position_ids_from_cu_seqlens(cu[: len(seqs) + 1], total))
        assert int(clean["num_real_tokens"]) == total == sum(lens_in)
        assert bool((base[total:] == tok.pad_token_id).all())


@settings(max_examples=80, deadline=None, derandomize=True)
@given(st.text(alphabet=LETTERS + LETTERS.lower() + "*- 1", max_size=120), st.integers(2, 64))
def test_tokenizers_are_total_and_respect_max_length(text, max_length):
    for tok in (ProtTokenizer(), StudentTokenizer()):
        ids = tok.encode(text)
        assert ids[-1] == tok.eos_token_id and all(0 <= i < tok.vocab_size for i in ids)
        assert len(ids) == len(tok._normalise(text)) + 1
        cut = tok(text, truncation=True, max_length=max_length)["input_ids"]
        assert len(cut) <= max_length and cut == ids[:len(cut) - 1] + [tok.eos_token_id] or len(ids) <= max_length
    assert ProtTokenizer().encode(text) == ProtTokenizer().encode(text.upper())  # case is normalised away


@settings(max_examples=30, deadline=None, derandomize=True)
@given(st.integers(1, 4), st.integers(1, 3), st.integers(1, 5), st.integers(0, 40), st.integers(0, 1000))
def test_balanced_sampler_partitions_each_epoch(world, accum, mbs, extra, seed):
    window = world * accum * mbs
    n = 3 * window + extra % window
    rng = np.random.default_rng(seed)
    lengths = rng.integers(5, 512, size=n)
    seen = []
    counts = set()
    for r in range(world):
        s = BalancedBatchSampler(lengths, mbs, accum, world=world, rank=r, seed=seed)
        s.set_epoch(1)
        batches = list(iter(s))
        counts.add(len(batches))
        assert len(batches) == len(s) == 3 * accum and all(len(b) == mbs for b in batches)
        seen += [i for b in batches for i in b]
    assert counts == {3 * accum} and len(seen) == len(set(seen)) == 3 * window      # nothing twice, whole windows only
    again = BalancedBatchSampler(lengths, mbs, accum, world=world, rank=0, seed=seed)
    again.set_epoch(1)
    again.fast_forward(accum)
    first = BalancedBatchSampler(lengths, mbs, accum, world=world, rank=0, seed=seed)
    first.set_epoch(1)
    assert list(iter(again)) == list(iter(first))[accum:]
