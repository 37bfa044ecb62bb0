"""The Fuji v3 (tiktoken-style, 128K) vocabulary: a Hugging Face ``tokenizers`` JSON file.

Counterpart of axlearn/experiments/text/gpt/vocabulary_fuji_v3.py (``FujiV3Vocabulary`` :75-225).
The file is looked up as ``<data_dir>/tokenizers/hf/<filename>`` (an absolute path is used as it
is).  ``encode`` never adds BOS or EOS; ``decode`` stops at the first EOS and drops BOS / padding.
Whole batches are encoded in one call into the tokenizer's native thread pool.
"""

from __future__ import annotations

import os
from typing import Optional, Sequence

from axlearn_b200.common.utils import get_data_dir


class FujiInnerTokenizer:
    """The piece-level view used by decoding-time logit modifiers."""

    def __init__(self, tokenizer):
        self._tokenizer = tokenizer

    def encode_as_pieces(self, text: str) -> list[str]:
        return self._tokenizer.encode(text, add_special_tokens=False).tokens

    def piece_to_id(self, piece: str) -> int:
        return self._tokenizer.token_to_id(piece)


class FujiV3Vocabulary:
    _PAD = ("<|pad_id|>", "<|finetune_right_pad_id|>")
    _EOS = "<|end_of_text|>"
    _BOS = "<|begin_of_text|>"

    def __init__(self, filename: str = "fuji-v3-tiktoken.json"):
        from tokenizers import Tokenizer  # pylint: disable=import-outside-toplevel

        if not os.path.isabs(filename):
            data_dir = get_data_dir()
            if data_dir in (None, "FAKE"):
                raise FileNotFoundError(f"{filename}: set a data directory holding tokenizers/hf/")
            filename = os.path.join(data_dir, "tokenizers", "hf", filename)
        self._tokenizer = Tokenizer.from_file(filename)
        self.vocab = self._tokenizer.get_vocab()
        self.tokenizer = FujiInnerTokenizer(self._tokenizer)

    @property
    def vocab_size(self) -> int:
        return self._tokenizer.get_vocab_size(with_added_tokens=True)

    def _special(self, names: Sequence[str], what: str) -> int:
        for name in names:
            if name in self.vocab:
                return self.vocab[name]
        raise ValueError(f"unable to infer the {what} token")

    @property
    def pad_id(self) -> int:
        return self._special(self._PAD, "pad")

    @property
    def eos_id(self) -> Optional[int]:
        return self._special((self._EOS,), "eos")

    @property
    def bos_id(self) -> Optional[int]:
        return self._special((self._BOS,), "bos")

    def _strip_bos(self, ids: list[int]) -> list[int]:
        bos = self.vocab.get(self._BOS)
        return ids[1:] if ids and ids[0] == bos else ids

    def encode(self, text: str) -> list[int]:
        return self._strip_bos(self._tokenizer.encode(text, add_special_tokens=True).ids)

    def encode_batch(self, texts: Sequence[str]) -> list[list[int]]:
        return [self._strip_bos(e.ids) for e in self._tokenizer.encode_batch(list(texts), add_special_tokens=True)]

    def _filtered(self, ids: Sequence[int]) -> list[int]:
        drop = {self.vocab.get(self._BOS), self.vocab.get(self._EOS)} | {self.vocab.get(p) for p in self._PAD}
        return [int(i) for i in ids if int(i) not in drop]

    def decode(self, ids: Sequence[int]) -> str:
        ids = [int(i) for i in ids]
        eos = self.vocab.get(self._EOS)
        if eos in ids:
            ids = ids[:ids.index(eos)]
        return self._tokenizer.decode(self._filtered(ids), skip_special_tokens=False)

    def decode_batch(self, batch: Sequence[Sequence[int]]) -> list[str]:
        return self._tokenizer.decode_batch([self._filtered(ids) for ids in batch], skip_special_tokens=False)
