"""SentencePiece training script (reference behaviour: axlearn/experiments/text/train_spm.py)."""

import json

import pytest

from axlearn_b200.common import tfrecord
from axlearn_b200.experiments.text import train_spm

spm = pytest.importorskip("sentencepiece")

_WORDS = "the quick brown fox jumps over the lazy dog while seven wizards quietly box small jumping frogs".split()


def _sentences(n, offset=0):
    return [" ".join(_WORDS[(i * 3 + j + offset) % len(_WORDS)] for j in range(5 + i % 7)) for i in range(n)]


def test_format_name_and_config_checks(tmp_path):
    assert train_spm.format_name("a/b/bpe_32k.json", "c4/en:3.0.1") == "spm_bpe_32k_c4_en_3_0_1"
    assert train_spm.format_name("bpe_32k.json") == "spm_bpe_32k"
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps({"pad_id": 0, "unk_id": 0, "eos_id": 1, "bos_id": -1}))
    with pytest.raises(ValueError, match="pad_id"):
        train_spm.build_spm_config("m", spm_config_file=str(bad), max_train_examples=10)
    ok = tmp_path / "ok.json"
    ok.write_text(json.dumps({"pad_id": 0, "eos_id": 1, "unk_id": 2, "bos_id": -1, "model_type": "bpe"}))
    cfg = train_spm.build_spm_config("m", spm_config_file=str(ok), max_train_examples=10)
    assert cfg["model_type"] == "bpe" and cfg["input_sentence_size"] == 10 and cfg["model_prefix"] == "m"


def test_shuffle_is_a_permutation():
    xs = [str(i) for i in range(100)]
    out = list(train_spm.shuffled(iter(xs), buffer_size=16, seed=1))
    assert sorted(out) == sorted(xs) and out != xs
    assert list(train_spm.shuffled(iter(xs), buffer_size=1, seed=1)) == xs


def test_train_from_mixed_corpus(tmp_path):
    (tmp_path / "a.jsonl").write_text("\n".join(json.dumps({"text": s}) for s in _sentences(200) + [""]) + "\n")
    (tmp_path / "b.txt").write_text("\n".join(_sentences(200, 1)) + "\n\n")
    with tfrecord.TFRecordWriter(str(tmp_path / "c.tfrecord")) as w:
        for s in _sentences(100, 2):
            w.write(tfrecord.encode_example({"text": s}))
    texts = list(train_spm.iter_texts(train_spm.expand_inputs([str(tmp_path / "*.jsonl"), str(tmp_path / "b.txt"),
                                                               str(tmp_path / "c.tfrecord")])))
    assert len(texts) == 500 and all(texts)
    cfg = tmp_path / "tiny_bpe.json"
    cfg.write_text(json.dumps({"pad_id": 0, "eos_id": 1, "unk_id": 2, "bos_id": -1, "vocab_size": 64,
                               "model_type": "bpe", "user_defined_symbols": "<n>", "num_threads": 1,
                               "train_extremely_large_corpus": False}))
    out_dir = tmp_path / "tok"
    args = train_spm.parser().parse_args(
        ["--input", str(tmp_path / "a.jsonl"), str(tmp_path / "b.txt"), str(tmp_path / "c.tfrecord"),
         "--spm_config_file", str(cfg), "--model_name", "toy", "--output_dir", str(out_dir), "--max_train_examples", "450"])
    model_file = train_spm.train(args)
    assert model_file == str(out_dir / "spm_tiny_bpe_toy.model")
    assert sorted(p.name for p in out_dir.iterdir()) == ["spm_tiny_bpe_toy.model", "spm_tiny_bpe_toy.vocab"]
    sp = spm.SentencePieceProcessor(model_file=model_file)
    assert sp.pad_id() == 0 and sp.eos_id() == 1 and sp.unk_id() == 2 and sp.get_piece_size() == 64
    assert sp.decode(sp.encode("the quick brown fox")) == "the quick brown fox"
    with pytest.raises(FileNotFoundError):
        train_spm.expand_inputs([str(tmp_path / "nothing*")])
