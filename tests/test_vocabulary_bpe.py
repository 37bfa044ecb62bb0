"""Byte-level BPE: training, round trips, agreement with transformers' GPT-2 tokenizer."""

import pytest

from axlearn_b200.common.input_lm import text_to_lm_training_input
from axlearn_b200.common.vocabulary_bpe import BPEVocabulary, bytes_to_unicode, train_bpe

CORPUS = ["the quick brown fox jumps over the lazy dog", "the lazy dog sleeps; the quick fox doesn't",
          "naïve café — 東京 2024!", "the the the quick quick"] * 3


def _vocab(tmp_path, size=300):
    vocab_file, merges_file = train_bpe(CORPUS, vocab_size=size, out_dir=str(tmp_path))
    return BPEVocabulary.default_config().set(vocab_file=vocab_file, merges_file=merges_file).instantiate()


def test_byte_map_is_a_bijection():
    m = bytes_to_unicode()
    assert len(m) == 256 and len(set(m.values())) == 256 and m[ord("a")] == "a" and m[ord(" ")] != " "


def test_train_encode_decode_round_trip(tmp_path):
    v = _vocab(tmp_path)
    assert 257 < v.vocab_size <= 300 and v.eos_id == v.vocab_size - 1 and v.pad_id == v.eos_id
    for text in CORPUS + ["unseen words: zebra ¿qué? 🙂", ""]:
        ids = v.encode(text)
        assert v.decode(ids) == text
    # Frequent words became single tokens (with their leading space).
    assert "Ġthe" in v.tokenize("over the hill") and "Ġquick" in v.tokenize("a quick one")
    assert len(v.encode("the quick")) < len("the quick".encode())
    # Merges never cross the pre-tokenisation boundaries.
    assert all(" " not in t and "Ġ" not in t[1:] for t in v.tokenize("the quick brown"))


def test_matches_the_tokenizers_library(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    v = _vocab(tmp_path)
    cfg = v.config
    ref = tokenizers.ByteLevelBPETokenizer(cfg.vocab_file, cfg.merges_file)
    for text in ["the quick brown fox doesn't sleep", "naïve café 2024!", "  two  spaces"]:
        assert v.encode(text) == ref.encode(text).ids


def test_feeds_the_lm_input_pipeline(tmp_path):
    v = _vocab(tmp_path)
    examples = list(text_to_lm_training_input([{"text": t} for t in CORPUS[:4]], vocab=v, max_len=16, window_size=4))
    assert examples and all(len(e["input_ids"]) == 16 for e in examples)
    assert examples[0]["input_ids"][0] == v.eos_id
