"""Amino-acid tokenizers implemented as numpy look-up tables (no HF tokenizers dependency).

ProtTokenizer reproduces the reference's 32-id vocabulary and text handling
(src/nanoplm/pretraining/models/modern_bert/tokenizer.py:20-62): ids 0..3 are <pad> </s> <unk>
<mask>, 4..28 are "ALGVSREDTIPKFQNYMHWCXBOUZ", 29 is <s>, 30/31 are unused; text is upper-cased,
U/Z/O/B become X, every character is one token, and the sequence is followed by </s> (and preceded
by <s> only with use_bos_token=True).

StudentTokenizer is the distillation student's 28-id vocabulary
(src/nanoplm/distillation/models/student/tokenizer.py): <pad> </s> <unk> then the 25 letters at
3..27, no mask token, no normalisation (lower case maps to <unk>).

TeacherTokenizer is the ProtT5 encoder's input convention
(src/nanoplm/distillation/models/teacher/prott5.py:67-70): upper-case, U/Z/O/B -> X, one token
per residue followed by </s>, in the 128-entry T5 sentencepiece id space.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Sequence

import numpy as np

AA_ORDER = "ALGVSREDTIPKFQNYMHWCXBOUZ"


class _LutTokenizer:
    pad_token, eos_token, unk_token = "<pad>", "</s>", "<unk>"
    pad_token_id, eos_token_id, unk_token_id = 0, 1, 2
    mask_token: str | None = None
    mask_token_id: int | None = None
    bos_token: str | None = None
    bos_token_id: int | None = None

    def __init__(self, vocab: dict[str, int]):
        self._vocab = dict(vocab)
        self._inv = {i: t for t, i in vocab.items()}
        self._lut = np.full(256, self.unk_token_id, dtype=np.uint8)
        for tok, idx in vocab.items():
            if len(tok) == 1:
                self._lut[ord(tok)] = idx

    # ---- vocabulary --------------------------------------------------------------------------
    def get_vocab(self) -> dict[str, int]:
        return dict(self._vocab)

    @property
    def vocab_size(self) -> int:
        return len(self._vocab)

    def __len__(self) -> int:
        return len(self._vocab)

    @property
    def all_special_ids(self) -> list[int]:
        ids = [self.pad_token_id, self.eos_token_id, self.unk_token_id]
        if self.mask_token_id is not None:
            ids.append(self.mask_token_id)
        if self.bos_token_id is not None:
            ids.append(self.bos_token_id)
        return sorted(set(ids))

    def convert_tokens_to_ids(self, tokens):
        if isinstance(tokens, str):
            return self._vocab.get(tokens, self.unk_token_id)
        return [self._vocab.get(t, self.unk_token_id) for t in tokens]

    def convert_ids_to_tokens(self, ids):
        if isinstance(ids, (int, np.integer)):
            return self._inv.get(int(ids), self.unk_token)
        return [self._inv.get(int(i), self.unk_token) for i in ids]

    def get_special_tokens_mask(self, ids: Sequence[int], already_has_special_tokens: bool = True):
        sp = set(self.all_special_ids)
        return [1 if int(i) in sp else 0 for i in ids]

    def special_mask_np(self, ids: np.ndarray) -> np.ndarray:
        lut = np.zeros(max(256, self.vocab_size), dtype=bool)
        lut[self.all_special_ids] = True
        return lut[ids]

    # ---- encoding ----------------------------------------------------------------------------
    def _normalise(self, text: str) -> bytes:
        return text.encode("ascii", errors="replace")

    def encode_np(self, text: str, add_special_tokens: bool = True, max_length: int | None = None,
                  truncation: bool = True) -> np.ndarray:
        raw = np.frombuffer(self._normalise(text), dtype=np.uint8)
        ids = self._lut[raw]
        if add_special_tokens:
            n_special = 1 + (self.bos_token_id is not None)
            if truncation and max_length is not None and len(ids) + n_special > max_length:
                # residues are cut, the special tokens stay (what the reference's HF tokenizer does:
                # a truncated sequence still ends in </s>)
                ids = ids[:max(0, max_length - n_special)]
            parts = []
            if self.bos_token_id is not None:
                parts.append(np.array([self.bos_token_id], dtype=np.uint8))
            parts.append(ids)
            parts.append(np.array([self.eos_token_id], dtype=np.uint8))
            ids = np.concatenate(parts)
        elif truncation and max_length is not None and len(ids) > max_length:
            ids = ids[:max_length]
        return ids

    def encode(self, text: str, add_special_tokens: bool = True, max_length: int | None = None,
               truncation: bool = True) -> list[int]:
        return self.encode_np(text, add_special_tokens, max_length, truncation).tolist()

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        sp = set(self.all_special_ids) if skip_special_tokens else set()
        return "".join(self._inv.get(int(i), self.unk_token) for i in ids if int(i) not in sp)

    def __call__(self, text, add_special_tokens: bool = True, max_length: int | None = None,
                 truncation: bool = False, padding=False, return_tensors: str | None = None, **_):
        single = isinstance(text, str)
        texts = [text] if single else list(text)
        enc = [self.encode_np(t, add_special_tokens, max_length, truncation) for t in texts]
        if padding or return_tensors is not None:
            width = max_length if padding == "max_length" and max_length else max(len(e) for e in enc)
            ids = np.full((len(enc), width), self.pad_token_id, dtype=np.int64)
            mask = np.zeros((len(enc), width), dtype=np.int64)
            for i, e in enumerate(enc):
                ids[i, :len(e)] = e
                mask[i, :len(e)] = 1
            if return_tensors == "pt":
                import torch
                return {"input_ids": torch.from_numpy(ids), "attention_mask": torch.from_numpy(mask)}
            out_ids, out_mask = ids.tolist(), mask.tolist()
        else:
            out_ids = [e.tolist() for e in enc]
            out_mask = [[1] * len(e) for e in enc]
        if single and return_tensors is None:
            return {"input_ids": out_ids[0], "attention_mask": out_mask[0]}
        return {"input_ids": out_ids, "attention_mask": out_mask}

    def batch_encode_plus(self, batch_text, **kwargs):
        """The HF spelling for a list of texts (the reference's distillation collator calls it,
        distillation/collator.py:49-68)."""
        return self(list(batch_text), **kwargs)

    def encode_plus(self, text: str, **kwargs):
        return self(text, **kwargs)

    def pad(self, examples: list[dict], return_tensors: str = "pt", **_):
        import torch
        width = max(len(e["input_ids"]) for e in examples)
        ids = torch.full((len(examples), width), self.pad_token_id, dtype=torch.long)
        mask = torch.zeros((len(examples), width), dtype=torch.long)
        for i, e in enumerate(examples):
            v = torch.as_tensor(e["input_ids"]).long()
            n = v.numel()
            if "attention_mask" in e:
                n = int(torch.as_tensor(e["attention_mask"]).sum())
            ids[i, :n] = v[:n]
            mask[i, :n] = 1
        return {"input_ids": ids, "attention_mask": mask}

    # ---- persistence (HF-style files so checkpoints carry a usable tokenizer) -------------------
    def save_pretrained(self, directory: str | Path) -> None:
        d = Path(directory)
        d.mkdir(parents=True, exist_ok=True)
        (d / "vocab.json").write_text(json.dumps(self._vocab, indent=2), encoding="utf-8")
        cfg = {"tokenizer_class": type(self).__name__, "pad_token": self.pad_token,
               "eos_token": self.eos_token, "unk_token": self.unk_token,
               "mask_token": self.mask_token, "bos_token": self.bos_token}
        (d / "tokenizer_config.json").write_text(json.dumps(cfg, indent=2), encoding="utf-8")

    def save_vocabulary(self, directory: str | Path, filename_prefix: str | None = None):
        d = Path(directory)
        d.mkdir(parents=True, exist_ok=True)
        name = (filename_prefix + "-" if filename_prefix else "") + "vocab.json"
        (d / name).write_text(json.dumps(self._vocab, indent=2), encoding="utf-8")
        return (str(d / name),)


class ProtTokenizer(_LutTokenizer):
    mask_token, mask_token_id = "<mask>", 3

    def __init__(self, use_bos_token: bool = False):
        vocab = {"<pad>": 0, "</s>": 1, "<unk>": 2, "<mask>": 3}
        for i, aa in enumerate(AA_ORDER):
            vocab[aa] = 4 + i
        vocab["<s>"] = 29
        vocab["<unused0>"] = 30
        vocab["<unused1>"] = 31
        super().__init__(vocab)
        self.use_bos_token = bool(use_bos_token)
        if use_bos_token:
            self.bos_token, self.bos_token_id = "<s>", 29
        # lower case maps like upper case; U Z O B are read as X
        for aa in AA_ORDER:
            self._lut[ord(aa.lower())] = self._lut[ord(aa)]
        for ch in "UZOBuzob":
            self._lut[ord(ch)] = self._vocab["X"]


class StudentTokenizer(_LutTokenizer):
    def __init__(self):
        vocab = {"<pad>": 0, "</s>": 1, "<unk>": 2}
        for i, aa in enumerate(AA_ORDER):
            vocab[aa] = 3 + i
        super().__init__(vocab)


# ProtT5 sentencepiece ids for single residues (spiece model order: frequency-sorted letters)
_T5_ORDER = "ALGVSREDTIPKFQNYMHWCXBOUZ"


class TeacherTokenizer(_LutTokenizer):
    """T5-encoder input ids: <pad>=0, </s>=1, <unk>=2, residues from 3, vocabulary padded to 128."""

    def __init__(self, vocab_size: int = 128):
        vocab = {"<pad>": 0, "</s>": 1, "<unk>": 2}
        for i, aa in enumerate(_T5_ORDER):
            vocab[aa] = 3 + i
        for i in range(len(vocab), vocab_size):
            vocab[f"<extra_id_{vocab_size - 1 - i}>"] = i
        super().__init__(vocab)
        for aa in _T5_ORDER:
            self._lut[ord(aa.lower())] = self._lut[ord(aa)]
        for ch in "UZOBuzob":
            self._lut[ord(ch)] = self._vocab["X"]

    @staticmethod
    def preprocess(seq: str) -> str:
        """The reference's text form: stripped, upper-cased, rare residues as X, space separated."""
        s = seq.strip().upper()
        for ch in "UZOB":
            s = s.replace(ch, "X")
        return " ".join(s)

    def _normalise(self, text: str) -> bytes:
        return text.replace(" ", "").encode("ascii", errors="replace")
