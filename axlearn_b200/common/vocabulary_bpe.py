"""Byte-level BPE vocabulary.

Parity target in the reference: axlearn/common/vocabulary_bpe.py (``BPEVocabulary``: a
byte-level BPE tokenizer defined by a ``vocab.json`` (token -> id) and a ``merges.txt`` (one merge
per line, most frequent first), GPT-2 conventions: bytes are mapped to printable unicode
characters, text is split by a regular expression before merging, so merges never cross word
boundaries).  ``train_bpe`` builds such files from raw text (small corpora; used by tests and
for quick experiments).
"""

from __future__ import annotations

import collections
import functools
import json
import os
from typing import Iterable, Optional, Sequence

import regex

from axlearn_b200.common.config import REQUIRED, Configurable, Required, config_class

_SPLIT = regex.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")


@functools.lru_cache(maxsize=1)
def bytes_to_unicode() -> dict[int, str]:
    """A reversible map from the 256 byte values to printable unicode characters (printable
    ASCII and Latin-1 keep their code points, the rest are shifted above 255)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    chars = keep[:]
    n = 0
    for b in range(256):
        if b not in keep:
            keep.append(b)
            chars.append(256 + n)
            n += 1
    return dict(zip(keep, map(chr, chars)))


def _merge_word(symbols: tuple, ranks: dict) -> tuple:
    """Applies merges to one pre-token, lowest rank (= earliest learned) first."""
    symbols = list(symbols)
    while len(symbols) > 1:
        best, best_rank = None, None
        for i in range(len(symbols) - 1):
            r = ranks.get((symbols[i], symbols[i + 1]))
            if r is not None and (best_rank is None or r < best_rank):
                best, best_rank = i, r
        if best is None:
            break
        pair = (symbols[best], symbols[best + 1])
        out, i = [], 0
        while i < len(symbols):
            if i < len(symbols) - 1 and (symbols[i], symbols[i + 1]) == pair:
                out.append(symbols[i] + symbols[i + 1])
                i += 2
            else:
                out.append(symbols[i])
                i += 1
        symbols = out
    return tuple(symbols)


class BPEVocabulary(Configurable):
    @config_class
    class Config(Configurable.Config):
        vocab_file: Required[str] = REQUIRED
        merges_file: Required[str] = REQUIRED
        eos_token: str = "<|endoftext|>"
        pad_token: Optional[str] = None
        unk_token: Optional[str] = None

    def __init__(self, cfg):
        super().__init__(cfg)
        with open(cfg.vocab_file, encoding="utf-8") as f:
            self._encoder: dict[str, int] = json.load(f)
        self._decoder = {i: t for t, i in self._encoder.items()}
        with open(cfg.merges_file, encoding="utf-8") as f:
            lines = [ln.rstrip("\n") for ln in f if ln.strip() and not ln.startswith("#version")]
        self._ranks = {tuple(ln.split(" ")): i for i, ln in enumerate(lines)}
        self._b2u = bytes_to_unicode()
        self._u2b = {u: b for b, u in self._b2u.items()}
        self._cache: dict[str, tuple] = {}

    @property
    def vocab_size(self) -> int:
        return len(self._encoder)

    @property
    def eos_id(self) -> int:
        return self._encoder[self._config.eos_token]

    @property
    def pad_id(self) -> int:
        cfg = self._config
        return self._encoder[cfg.pad_token] if cfg.pad_token is not None else self.eos_id

    def tokenize(self, text: str) -> list[str]:
        out = []
        for piece in _SPLIT.findall(text):
            word = "".join(self._b2u[b] for b in piece.encode("utf-8"))
            merged = self._cache.get(word)
            if merged is None:
                merged = self._cache[word] = _merge_word(tuple(word), self._ranks)
            out.extend(merged)
        return out

    def encode(self, text: str) -> list[int]:
        cfg = self._config
        ids = []
        for tok in self.tokenize(text):
            if tok in self._encoder:
                ids.append(self._encoder[tok])
            elif cfg.unk_token is not None:
                ids.append(self._encoder[cfg.unk_token])
            else:
                raise KeyError(f"token {tok!r} is not in the vocabulary and no unk_token is configured")
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        special = {self._config.eos_token, self._config.pad_token, self._config.unk_token}
        text = "".join(self._decoder[int(i)] for i in ids if self._decoder.get(int(i)) not in special)
        return bytes(self._u2b[c] for c in text).decode("utf-8", errors="replace")


def train_bpe(texts: Iterable[str], *, vocab_size: int, out_dir: str, eos_token: str = "<|endoftext|>") -> tuple[str, str]:
    """Learns merges until the vocabulary (256 byte symbols + merges + eos) has ``vocab_size``
    entries; writes ``vocab.json`` / ``merges.txt`` into ``out_dir`` and returns their paths."""
    b2u = bytes_to_unicode()
    words = collections.Counter()
    for text in texts:
        for piece in _SPLIT.findall(text):
            words[tuple(b2u[b] for b in piece.encode("utf-8"))] += 1
    vocab = [b2u[b] for b in range(256)]
    merges = []
    while len(vocab) + 1 < vocab_size:
        pairs = collections.Counter()
        for word, n in words.items():
            for a, b in zip(word, word[1:]):
                pairs[(a, b)] += n
        if not pairs:
            break
        (a, b), count = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        if count < 2:
            break
        merges.append((a, b))
        vocab.append(a + b)
        ranks = {(a, b): 0}
        words = collections.Counter({_merge_word(w, ranks): n for w, n in words.items()})
    vocab.append(eos_token)
    os.makedirs(out_dir, exist_ok=True)
    vocab_file, merges_file = os.path.join(out_dir, "vocab.json"), os.path.join(out_dir, "merges.txt")
    with open(vocab_file, "w", encoding="utf-8") as f:
        json.dump({t: i for i, t in enumerate(vocab)}, f, ensure_ascii=False)
    with open(merges_file, "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n")
    return vocab_file, merges_file
