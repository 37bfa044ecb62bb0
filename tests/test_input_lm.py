"""Text -> LM inputs: packing, masking variants, eval windows, prefixes, batching and resume."""

import torch

from axlearn_b200.common import input_lm
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.input_lm import ByteVocabulary, PackingMethodType, TextLmInput

VOCAB = ByteVocabulary.default_config().instantiate()
DOCS = [{"text": "hello world"}, {"text": "ab"}, {"text": "the quick brown fox"}, {"text": "z" * 7}]


def _stream():
    out = [VOCAB.eos_id]
    for d in DOCS:
        out += VOCAB.encode(d["text"]) + [VOCAB.eos_id]
    return out


def test_byte_vocabulary_roundtrip():
    ids = VOCAB.encode("héllo")
    assert VOCAB.decode(ids) == "héllo" and min(ids) >= 3 and VOCAB.vocab_size == 259


def test_training_input_packs_the_concatenated_stream():
    exs = list(input_lm.text_to_lm_training_input(DOCS, vocab=VOCAB, max_len=16, window_size=10))
    stream = _stream()
    n = len(stream) - 1
    assert len(exs) == -(-n // 16)          # the padded tail is kept with max_padding_fraction = 1
    flat_in = [t for e in exs for t in e["input_ids"]][:n]
    flat_tg = [t for e in exs for t in e["target_labels"]][:n]
    assert flat_in == stream[:-1] and flat_tg == stream[1:]
    assert all(len(e["input_ids"]) == 16 and len(e["target_labels"]) == 16 for e in exs)
    assert exs[-1]["target_labels"][n - 16 * (len(exs) - 1):] == [0] * (16 * len(exs) - n)
    total_bytes = sum(e["target_num_bytes"] for e in exs)
    assert total_bytes == sum(len(d["text"]) for d in DOCS)
    # A tail that would need too much padding is dropped.
    strict = list(input_lm.text_to_lm_training_input(DOCS, vocab=VOCAB, max_len=16, window_size=10,
                                                     max_padding_fraction=0.0))
    assert len(strict) == n // 16


def test_training_input_with_segment_masking():
    exs = list(input_lm.text_to_lm_training_input(
        DOCS, vocab=VOCAB, max_len=16, window_size=10, packing_method=PackingMethodType.EOS_DELIM_MASK))
    first = exs[0]
    seg, pos = first["input_segment_ids"], first["input_positions"]
    assert seg[0] == 1 and pos[0] == 0
    for i in range(1, 16):
        if seg[i] == 0:
            continue
        if seg[i] == seg[i - 1]:
            assert pos[i] == pos[i - 1] + 1
        else:
            assert seg[i] == seg[i - 1] + 1 and pos[i] == 0
    # "hello world" is 11 bytes: the leading EOS is its own segment, then 12 tokens of document 1.
    assert seg[:14] == [1] + [2] * 12 + [3]


def test_shuffle_is_seeded_and_complete():
    kw = dict(vocab=VOCAB, max_len=8, window_size=2)
    plain = list(input_lm.text_to_lm_training_input(DOCS, **kw))
    a = list(input_lm.text_to_lm_training_input(DOCS, shuffle_buffer_size=4, seed=1, **kw))
    b = list(input_lm.text_to_lm_training_input(DOCS, shuffle_buffer_size=4, seed=1, **kw))
    assert a == b and a != plain
    assert sorted(map(str, a)) == sorted(map(str, plain))


def test_eval_input_scores_every_token_once():
    doc = [{"text": "abcdefghijklmnopqrstuvwxyz"}]
    exs = list(input_lm.text_to_lm_eval_input(doc, vocab=VOCAB, max_len=8, stride=4))
    live = [t for e in exs for t in e["target_labels"] if t != 0]
    assert live == VOCAB.encode(doc[0]["text"]) + [VOCAB.eos_id]
    assert sum(e["target_num_bytes"] for e in exs) == 26
    # Later windows carry context: their first targets are masked out.
    assert exs[1]["target_labels"][:4] == [0, 0, 0, 0] and exs[1]["input_ids"][0] != 0


def test_decoding_prefix_processor():
    (ex,) = list(input_lm.lm_decoding_prefix_processor([{"text": "hi"}], vocab=VOCAB, max_len=6))
    assert ex["prefix"] == [1] + VOCAB.encode("hi") + [0, 0, 0]


def _input(**kw):
    proc = lambda src: input_lm.text_to_lm_training_input(src, vocab=VOCAB, max_len=8, window_size=2)
    return TextLmInput.default_config().set(
        name="input", global_batch_size=2, source=lambda: iter(DOCS), processor=proc, **kw).instantiate(parent=None)


def test_text_lm_input_batches_repeat_and_resume():
    inp = _input(total_num_batches=5)
    batches = list(inp.dataset())
    assert len(batches) == 5 and batches[0]["input_ids"].shape == (2, 8)
    assert batches[0]["input_ids"].dtype == torch.int32
    # A fresh input positioned after two batches continues with the third.
    resumed = _input(total_num_batches=5)
    resumed.set_state({"batch_index": 2})
    rest = list(resumed.dataset())
    assert len(rest) == 3 and torch.equal(rest[0]["input_ids"], batches[2]["input_ids"])
    # Feeds partition the rows of the same global batch.
    f0 = next(iter(_input(num_feeds=2, feed_index=0).dataset()))
    f1 = next(iter(_input(num_feeds=2, feed_index=1).dataset()))
    assert torch.equal(torch.cat([f0["input_ids"], f1["input_ids"]]), batches[0]["input_ids"])
