"""Text preprocessing processors.

Parity target: axlearn/common/input_text.py -- ``preprocess_chunks`` :69, ``strip_accents`` :103,
``tokenize`` :134, ``add_token_type_ids`` :161, ``tokenize_example`` :228, ``num_bytes`` :249,
``pack_strings`` / ``unpack_strings`` :278-335, ``infer_bos_id`` :337, ``roberta_normalize`` :356,
``bert_normalize`` :395-466, ``split_sentences`` :469, ``random_chunking`` :515,
``join_string_features`` :543 -- and the Grain text helpers (axlearn/common/input_grain_text.py:
``with_regex_mapping`` :48, ``tokenize`` :100, ``num_bytes`` :146, ``count_num_bytes`` :178).

All processors are ``DatasetToDatasetFn`` over iterables of dict examples (see
``input_processing``); strings are Python ``str`` and ids numpy int32 arrays.  A vocabulary is
anything with ``encode(str) -> ids``, ``decode(ids) -> str``, ``eos_id``, ``pad_id`` and
(optionally) ``bos_id``.
"""

from __future__ import annotations

import re
import unicodedata
from typing import Any, Callable, Iterator, Optional, Sequence, Union

import numpy as np

from axlearn_b200.common.config import ConfigOr, maybe_instantiate
from axlearn_b200.common.input_processing import Dataset, DatasetToDatasetFn, Example, map_over_dataset

INPUT_IDS = "input_ids"
TOKEN_TYPE_IDS = "token_type_ids"
STRINGS_BYTE_ARRAY_PAD_VALUE = np.iinfo(np.int32).max


def _as_keys(key: Union[str, Sequence[str]]) -> list:
    return [key] if isinstance(key, str) else list(key)


def preprocess_chunks(chunk_size: int) -> DatasetToDatasetFn:
    """One example per ``chunk_size`` characters of every document's "text"."""

    def process(ds: Dataset) -> Iterator[Example]:
        for ex in ds:
            text = ex["text"]
            for k in range(0, len(text), chunk_size):
                yield {"text": text[k: k + chunk_size]}

    return process


def _strip_marks(text: str) -> str:
    return "".join(c for c in text if unicodedata.category(c) != "Mn")


def strip_accents(fields: Sequence[str], normalization_form: str = "NFKD") -> DatasetToDatasetFn:
    if normalization_form not in ("NFD", "NFKD"):
        raise ValueError(normalization_form)

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for f in fields:
            ex[f] = _strip_marks(unicodedata.normalize(normalization_form, ex[f]))
        return ex

    return map_over_dataset(fn)


def tokenize_example(text: str, vocab: Any, replace_newlines_with: str = "\n") -> np.ndarray:
    """Ids of ``text`` without padding or BOS / EOS."""
    return np.asarray(vocab.encode(text.replace("\n", replace_newlines_with)), dtype=np.int32)


def tokenize(output_features: ConfigOr[dict], *, copy_pretokenized: bool = True, with_eos: bool = False,
             replace_newlines_with: str = "\n") -> DatasetToDatasetFn:
    """``output_features``: ``{field: vocab}`` or ``{field: {"vocab": v, "add_eos": bool}}``.  String
    fields named there are replaced by their ids; with ``copy_pretokenized`` the text stays under
    ``<field>_pretokenized``."""
    feats = maybe_instantiate(output_features)

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for key, feat in feats.items():
            if key not in ex or not isinstance(ex[key], str):
                continue
            vocab, add_eos = (feat["vocab"], feat.get("add_eos", with_eos)) if isinstance(feat, dict) else (feat, with_eos)
            text = ex[key]
            if copy_pretokenized:
                ex[f"{key}_pretokenized"] = text
            ids = tokenize_example(text, vocab, replace_newlines_with)
            if add_eos:
                ids = np.concatenate([ids, np.asarray([vocab.eos_id], dtype=np.int32)])
            ex[key] = ids
        return ex

    return map_over_dataset(fn)


def add_token_type_ids(input_key: Union[str, Sequence[str]], output_key: str = TOKEN_TYPE_IDS) -> DatasetToDatasetFn:
    """Type id ``i`` for the tokens of the i-th sequence and the separator / EOS after it; BOS has
    type 0.  (``[BOS] a [SEP] b [EOS]`` -> ``0 0.. 0 1.. 1``.)"""
    keys = _as_keys(input_key)

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        parts = []
        for i, key in enumerate(keys):
            t = np.asarray(ex[key])
            parts.append(np.full(t.shape[:-1] + (int(i == 0) + t.shape[-1] + 1,), i, dtype=np.int32))
        ex[output_key] = np.concatenate(parts, axis=-1)
        return ex

    return map_over_dataset(fn)


def num_bytes(ids: Any, vocab: Any, newlines_replaced_with: str = "\n") -> Any:
    """UTF-8 bytes of the decoded ids, every EOS counting one byte.  1-D ids -> int; 2-D -> [B]."""
    a = np.asarray(ids)
    if a.ndim == 2:
        return np.asarray([num_bytes(r, vocab, newlines_replaced_with) for r in a], dtype=np.int32)
    eos = getattr(vocab, "eos_id", None)
    pad = getattr(vocab, "pad_id", None)
    body = [int(t) for t in a if t != eos and t != pad]
    text = vocab.decode(body).replace(newlines_replaced_with, "\n") if newlines_replaced_with != "\n" else vocab.decode(body)
    return len(text.encode("utf-8")) + int((a == eos).sum())


def count_num_bytes(*, input_key: str, vocab: Any, output_key: Optional[str] = None) -> DatasetToDatasetFn:
    out = output_key or f"{input_key}_num_bytes"

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        ex[out] = num_bytes(ex[input_key], vocab)
        return ex

    return map_over_dataset(fn)


def pack_strings(strings: Sequence[str], max_packed_byte_array_len: int) -> np.ndarray:
    """``[len(strings), max_len]`` int32 code points padded with ``STRINGS_BYTE_ARRAY_PAD_VALUE`` --
    a fixed-shape form of strings that a collective can carry between processes."""
    out = np.full((len(strings), max_packed_byte_array_len), STRINGS_BYTE_ARRAY_PAD_VALUE, dtype=np.int32)
    for i, s in enumerate(strings):
        if isinstance(s, bytes):
            s = s.decode("utf-8")
        cps = [ord(c) for c in s]
        if len(cps) > max_packed_byte_array_len:
            raise ValueError(f"string {i} has {len(cps)} code points > {max_packed_byte_array_len}")
        out[i, : len(cps)] = cps
    return out


def unpack_strings(strings_byte_array: Any) -> list:
    a = np.asarray(strings_byte_array)
    return ["".join(chr(int(c)) for c in row[row != STRINGS_BYTE_ARRAY_PAD_VALUE]) for row in a]


def infer_bos_id(vocab: Any) -> int:
    """BOS of the vocabulary, or EOS when it has none."""
    bos = getattr(vocab, "bos_id", None)
    if bos is None or bos < 0:
        bos = getattr(vocab, "eos_id", None)
    if bos is None or bos < 0:
        raise ValueError(f"Cannot infer a viable bos_id from vocabulary: {vocab}")
    return int(bos)


def roberta_normalize(cased: bool = True, input_key: Union[str, Sequence[str]] = "text") -> DatasetToDatasetFn:
    keys = _as_keys(input_key)

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for k in keys:
            t = ex[k]
            ex[k] = (t if cased else t.lower()).strip()
        return ex

    return map_over_dataset(fn)


def _is_punct(c: str) -> bool:
    cp = ord(c)
    if 33 <= cp <= 47 or 58 <= cp <= 64 or 91 <= cp <= 96 or 123 <= cp <= 126:
        return True
    return unicodedata.category(c).startswith("P")


def _is_cjk(c: str) -> bool:
    cp = ord(c)
    return (0x4E00 <= cp <= 0x9FFF or 0x3400 <= cp <= 0x4DBF or 0x20000 <= cp <= 0x2A6DF or 0x2A700 <= cp <= 0x2B73F
            or 0x2B740 <= cp <= 0x2B81F or 0x2B820 <= cp <= 0x2CEAF or 0xF900 <= cp <= 0xFAFF or 0x2F800 <= cp <= 0x2FA1F)


def bert_basic_tokenize(text: str, *, lower_case: bool) -> list:
    """BERT's basic tokeniser without accent stripping: drop NUL / U+FFFD / control and combining
    marks, normalise whitespace, isolate CJK characters and punctuation."""
    out: list = []
    word: list = []

    def flush():
        if word:
            out.append("".join(word))
            word.clear()

    for c in text:
        cp = ord(c)
        cat = unicodedata.category(c)
        if cp == 0 or cp == 0xFFFD or cat == "Mn":
            continue
        if c in "\t\n\r" or cat == "Zs" or c == " ":
            flush()
        elif cat.startswith("C"):
            continue
        elif _is_cjk(c) or _is_punct(c):
            flush()
            out.append(c)
        else:
            word.append(c.lower() if lower_case else c)
    flush()
    return out


def bert_normalize_mapper(cased: bool = True, input_key: Union[str, Sequence[str]] = "text") -> Callable[[Example], Example]:
    keys = _as_keys(input_key)

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for k in keys:
            ex[k] = " ".join(bert_basic_tokenize(ex[k], lower_case=not cased))
        return ex

    return fn


def bert_normalize(cased: bool = True, input_key: Union[str, Sequence[str]] = "text") -> DatasetToDatasetFn:
    return map_over_dataset(bert_normalize_mapper(cased=cased, input_key=input_key))


_SENTENCE_END = re.compile(r"(?<=[.!?])[\"')\]]*\s+(?=[\"'(\[]*[A-Z0-9a-z])")
_ABBREVIATIONS = {"mr.", "mrs.", "ms.", "dr.", "prof.", "sr.", "jr.", "st.", "vs.", "etc.", "e.g.", "i.e.", "inc.", "ltd.",
                  "co.", "no.", "fig.", "u.s."}


def sentence_split(text: str) -> list:
    """Rule-based sentence boundaries: ``. ! ?`` (with trailing quotes / brackets) followed by
    whitespace, except after common abbreviations and single initials."""
    sentences, start = [], 0
    for m in _SENTENCE_END.finditer(text):
        head = text[start: m.start()].rstrip("\"')]")
        last = head.split()[-1].lower() if head.split() else ""
        if last in _ABBREVIATIONS or (len(last) == 2 and last[0].isalpha() and last[1] == "."):
            continue
        sentences.append(text[start: m.end()].strip())
        start = m.end()
    tail = text[start:].strip()
    if tail:
        sentences.append(tail)
    return sentences


def split_sentences(input_key: str = "text", max_sentences_per_example: Optional[int] = None,
                    passthrough_keys: Optional[Sequence[str]] = None, *, seed: int = 0) -> DatasetToDatasetFn:
    """One (lower-cased) example per sentence, plus an empty sentence after every document."""
    passthrough_keys = list(passthrough_keys or [])

    def process(ds: Dataset) -> Iterator[Example]:
        rng = np.random.default_rng(seed)
        for ex in ds:
            sentences = sentence_split(ex[input_key].lower())
            if max_sentences_per_example is not None and len(sentences) > max_sentences_per_example > 0:
                idx = np.sort(rng.choice(len(sentences), size=max_sentences_per_example, replace=False))
                sentences = [sentences[i] for i in idx]
            for s in sentences + [""]:
                out = {input_key: s}
                for k in passthrough_keys:
                    out[k] = ex[k]
                yield out

    return process


def random_chunking(max_len: int, input_key: str = INPUT_IDS, *, seed: int = 0) -> DatasetToDatasetFn:
    """A uniformly placed window of ``min(len, max_len)`` ids."""

    def process(ds: Dataset) -> Iterator[Example]:
        rng = np.random.default_rng(seed)
        for ex in ds:
            ex = dict(ex)
            ids = np.asarray(ex[input_key])
            offset = int(rng.integers(0, max(0, len(ids) - max_len) + 1))
            ex[input_key] = ids[offset: offset + max_len]
            yield ex

    return process


def join_string_features(features: Sequence[str], key: str, separator: str = "</s>") -> DatasetToDatasetFn:
    def fn(ex: Example) -> Example:
        ex = dict(ex)
        ex[key] = separator.join(ex[f] for f in features)
        return ex

    return map_over_dataset(fn)


def with_regex_mapping(vocab_cls: type, *, encode_mapping: Sequence[tuple], decode_mapping: Sequence[tuple]) -> type:
    """A subclass of ``vocab_cls`` that rewrites text with ``(pattern, replacement)`` pairs before
    encoding and after decoding (e.g. newline <-> a reserved piece)."""
    enc = [(re.compile(p), r) for p, r in encode_mapping]
    dec = [(re.compile(p), r) for p, r in decode_mapping]

    class _Mapped(vocab_cls):  # type: ignore[misc, valid-type]
        def encode(self, s: str):
            for p, r in enc:
                s = p.sub(r, s)
            return super().encode(s)

        def decode(self, ids):
            s = super().decode(ids)
            for p, r in dec:
                s = p.sub(r, s)
            return s

    _Mapped.__name__ = f"RegexMapped{vocab_cls.__name__}"
    return _Mapped
