"""MLM corruption on numpy / torch arrays.

Semantics of the reference collators (src/nanoplm/pretraining/collator.py:54-111, 333-382):
Bernoulli(mlm_probability) selects positions among non-special, non-padding tokens; labels are the
original ids there and -100 elsewhere; one uniform draw per position picks <mask> / random token /
keep with the three proportions normalised to sum to one; random replacements come from the
vocabulary minus special ids.
"""
from __future__ import annotations

import numpy as np


class MLMMasker:
    def __init__(self, tokenizer, mlm_probability: float = 0.3, mask_token_probability: float = 0.8,
                 random_token_probability: float = 0.1, keep_probability: float = 0.1,
                 extra_excluded_token_ids=None):
        if getattr(tokenizer, "mask_token_id", None) is None:
            raise ValueError("Tokenizer must define a mask_token_id for MLM.")
        total = mask_token_probability + random_token_probability + keep_probability
        if total <= 0:
            raise ValueError("mask/random/keep probabilities must sum to a positive value")
        self.mlm_probability = float(mlm_probability)
        self.p_mask = mask_token_probability / total
        self.p_rand = random_token_probability / total
        self.p_keep = keep_probability / total
        self.mask_token_id = int(tokenizer.mask_token_id)
        special = set(tokenizer.all_special_ids)
        special.add(self.mask_token_id)
        if extra_excluded_token_ids:
            special.update(int(i) for i in extra_excluded_token_ids)
        allowed = [i for i in tokenizer.get_vocab().values() if i not in special]
        if not allowed:
            raise ValueError("No allowable token ids for random replacement after exclusions.")
        self.allowed_random_token_ids = np.asarray(sorted(allowed), dtype=np.int64)
        n = max(256, max(tokenizer.get_vocab().values()) + 1)
        self._special_lut = np.zeros(n, dtype=bool)
        self._special_lut[list(tokenizer.all_special_ids)] = True

    def special_mask(self, ids: np.ndarray) -> np.ndarray:
        return self._special_lut[ids]

    def __call__(self, ids: np.ndarray, rng: np.random.Generator, forbid: np.ndarray | None = None):
        """ids: int64 array (any shape). Returns (corrupted ids, labels); inputs are not modified."""
        ids = np.asarray(ids, dtype=np.int64)
        blocked = self.special_mask(ids)
        if forbid is not None:
            blocked = blocked | forbid
        selected = (rng.random(ids.shape) < self.mlm_probability) & ~blocked
        labels = np.where(selected, ids, -100)
        dice = rng.random(ids.shape)
        to_mask = selected & (dice < self.p_mask)
        to_rand = selected & (dice >= self.p_mask) & (dice < self.p_mask + self.p_rand)
        out = ids.copy()
        out[to_mask] = self.mask_token_id
        n_rand = int(to_rand.sum())
        if n_rand:
            out[to_rand] = self.allowed_random_token_ids[
                rng.integers(0, len(self.allowed_random_token_ids), size=n_rand)]
        return out, labels
