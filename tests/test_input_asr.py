"""ASR input processors (golden values: axlearn/audio/input_asr_test.py:22-101)."""

import numpy as np
import pytest

from axlearn_b200.audio import input_asr

_SPEECH = [[-29515.0, -18256.0], [14620.0, -21206.0, -4254.0], [-3954.0, -15555.0, 18074.0, 22466.0]]


class _CharVocab:
    eos_id = 1
    vocab_size = 128

    def encode(self, text):
        return [ord(c) for c in text]


def _run(processor, examples):
    return list(processor(iter(examples)))


@pytest.mark.parametrize("kw,want", [
    (dict(max_len=5), [([-29515.0, -18256.0, 0, 0, 0], [0, 0, 1, 1, 1]), ([14620.0, -21206.0, -4254.0, 0, 0], [0, 0, 0, 1, 1]),
                       ([-3954.0, -15555.0, 18074.0, 22466.0, 0], [0, 0, 0, 0, 1])]),
    (dict(max_len=2), [([-29515.0, -18256.0], [0, 0])]),
    (dict(max_len=2, truncate=True), [([-29515.0, -18256.0], [0, 0]), ([14620.0, -21206.0], [0, 0]), ([-3954.0, -15555.0], [0, 0])]),
    (dict(max_len=5, normalize_by_scale=2**15),
     [([-0.9007263, -0.5571289, 0.0, 0.0, 0.0], [0, 0, 1, 1, 1]), ([0.446167, -0.64715576, -0.12982178, 0.0, 0.0], [0, 0, 0, 1, 1]),
      ([-0.1206665, -0.47470093, 0.5515747, 0.6856079, 0.0], [0, 0, 0, 0, 1])]),
    (dict(max_len=2, normalize_by_scale=2**15, input_key="input_speech"), [([-0.9007263, -0.5571289], [0, 0])]),
])
def test_speech_input(kw, want):
    key = kw.get("input_key", "speech")
    out = _run(input_asr.speech_input(**kw), [{key: np.asarray(s), "id": i} for i, s in enumerate(_SPEECH)] + [{key: np.zeros([0])}])
    assert len(out) == len(want)
    for got, (inputs, paddings) in zip(out, want):
        assert got["inputs"].dtype == np.float32 and got["paddings"].dtype == bool and key not in got and "id" in got
        np.testing.assert_allclose(got["inputs"], inputs, rtol=1e-6)
        assert got["paddings"].astype(int).tolist() == paddings
    with pytest.raises(ValueError):
        input_asr.speech_input(max_len=0)
    with pytest.raises(ValueError):
        input_asr.speech_input(max_len=2, normalize_by_scale=-1.0)


def test_text_input_and_autoregressive_inputs():
    vocab = _CharVocab()
    exs = [{"text": "ab"}, {"text": ""}, {"text": "abcd"}, {"text": "abcde"}]
    out = _run(input_asr.text_input(max_len=5, vocab=vocab, truncate=False), exs)
    # "" is too short; "abcde" + EOS would not fit.
    assert [e["text"] for e in out] == ["ab", "abcd"]
    assert out[0]["target_labels"].tolist() == [97, 98, 1, -1, -1] and out[1]["target_labels"].tolist() == [97, 98, 99, 100, 1]
    out = _run(input_asr.text_input(max_len=5, vocab=vocab, truncate=True, eos_id=7), exs)
    assert [e["target_labels"].tolist() for e in out] == [[97, 98, 7, -1, -1], [97, 98, 99, 100, 7], [97, 98, 99, 100, 101]]
    assert len(_run(input_asr.text_input(max_len=5, vocab=vocab, truncate=True, min_len=3), exs)) == 2

    ar = _run(input_asr.make_autoregressive_inputs(vocab=vocab, bos_id=2), out[:1])
    assert ar[0]["input_ids"].tolist() == [2, 97, 98, 7, -1]
    ar = _run(input_asr.make_autoregressive_inputs(vocab=vocab, bos_id=None), out[:1])
    assert ar[0]["input_ids"][0] == 128


def test_pad_example():
    ex = {"source": {"inputs": np.ones([4], np.float32), "paddings": np.zeros([4], bool)},
          "target": {"input_ids": np.arange(3, dtype=np.int32)}, "target_labels": np.arange(3, dtype=np.int32)}
    pad = input_asr.pad_example_fn(ex)
    assert pad["source"]["paddings"].all() and not pad["source"]["inputs"].any()
    assert pad["target"]["input_ids"].tolist() == [-1] * 3 and pad["target_labels"].tolist() == [-1] * 3
