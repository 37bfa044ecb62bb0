"""Dataset processors, composite inputs, ranking and GLUE preprocessing (CPU)."""

import numpy as np
import pytest

from axlearn_b200.common import input_glue, input_processing as ip, input_text
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.input_composite import ConcatenatedInput, ZipInput
from axlearn_b200.common.input_ranking import rank_by_value


def _range_source(n, key="x"):
    return lambda: ({key: np.int32(i)} for i in range(n))


class _Vocab:
    """Whitespace vocabulary: every distinct word gets an id >= 3; 0 pad, 1 eos, 2 bos."""
    pad_id, eos_id, bos_id = 0, 1, 2

    def __init__(self):
        self.words = {}

    def encode(self, s):
        return [self.words.setdefault(w, len(self.words) + 3) for w in s.split()]

    def decode(self, ids):
        inv = {v: k for k, v in self.words.items()}
        return " ".join(inv[int(i)] for i in ids)


def test_chain_rekey_select_remove_filter():
    ds = [{"a": 1, "b": {"c": 2}}, {"a": 3, "b": {"c": 4}}]
    out = list(ip.chain(ip.rekey({"x": "a", "y": "b/c", "z": None}, default_value=-1, separator="/"),
                        ip.filter_examples(lambda e: e["x"] > 1))(ds))
    assert out == [{"x": 3, "y": 4, "z": -1}]
    assert list(ip.rekey({"x": "missing"}, default_value=None)(ds)) == [{}, {}]
    assert list(ip.rekey({"x": "a"}, retain_original_inputs=True)(ds))[0] == {"a": 1, "b": {"c": 2}, "x": 1}
    assert list(ip.select_fields(["a"])(ds)) == [{"a": 1}, {"a": 3}]
    assert list(ip.remove_fields(["b"])(ds)) == [{"a": 1}, {"a": 3}]
    assert list(ip.unpack({"c": ("b", "c")})(ds))[1]["c"] == 4
    assert list(ip.add_static_fields({"k": "v"})(ds))[0]["k"] == "v"
    assert list(ip.extract_from_sequence("s", "first")([{"s": [7, 8]}]))[0]["first"] == 7


def test_unbatch_take_shuffle_concat_sample():
    ds = [{"x": np.arange(3)}, {"x": np.arange(3, 5)}]
    assert [int(e["x"]) for e in ip.unbatch()(ds)] == [0, 1, 2, 3, 4]
    assert len(list(ip.take(2)(ip.unbatch()(ds)))) == 2
    shuffled = [int(e["x"]) for e in ip.shuffle(4, seed=1)(_range_source(20)())]
    assert sorted(shuffled) == list(range(20)) and shuffled != list(range(20))
    assert shuffled == [int(e["x"]) for e in ip.shuffle(4, seed=1)(_range_source(20)())]
    cat = ip.concatenate_datasets(sources=[_range_source(2), _range_source(3)])
    assert [int(e["x"]) for e in cat()] == [0, 1, 0, 1, 2]

    def forever(v):
        def fn():
            while True:
                yield {"x": v}
        return fn

    mix = ip.sample_from_datasets(sources=[forever(0), forever(1), forever(2)], weights=[0.75, 0.25, 0.0], seed=0)
    draws = [e["x"] for e in ip.take(2000)(mix())]
    assert 2 not in draws and abs(np.mean(np.asarray(draws) == 0) - 0.75) < 0.05
    with pytest.raises(ValueError):
        ip.sample_from_datasets(sources=[forever(0)], weights=[0.0])


def test_skip_on_error():
    def bad():
        for i in range(5):
            yield {"x": i}

    class Flaky:
        def __iter__(self):
            self.i = 0
            return self

        def __next__(self):
            self.i += 1
            if self.i > 5:
                raise StopIteration
            if self.i % 2 == 0:
                raise ValueError("decode")
            return {"x": self.i}

    assert [e["x"] for e in ip.skip_on_error()(Flaky())] == [1, 3, 5]
    assert len(list(ip.skip_on_error()(bad()))) == 5


def test_trim_pad_pack():
    assert ip.trim_and_pad_tensor([1, 2, 3], 5, pad_id=9).tolist() == [1, 2, 3, 9, 9]
    assert ip.trim_and_pad_tensor(np.ones((2, 6)), 4).shape == (2, 4)
    padded = list(ip.pad_to_batch(4)([{"x": np.ones((3, 2))}]))[0]["x"]
    assert padded.shape == (4, 2) and padded[3].sum() == 0
    with pytest.raises(ValueError):
        list(ip.pad_to_batch(2)([{"x": np.ones((3, 2))}]))
    assert list(ip.trim_to_batch(2)([{"x": np.arange(5)}]))[0]["x"].tolist() == [0, 1]
    rows = [{"x": np.full((n, 1), n)} for n in (2, 1, 3, 2, 2)]
    packed = [e["x"][:, 0].tolist() for e in ip.pack_to_batch(4)(rows)]
    assert packed == [[2, 2, 1, 0], [3, 3, 3, 0], [2, 2, 2, 2]]
    with pytest.raises(ValueError):
        list(ip.pack_to_batch(2)([{"x": np.ones((3, 1))}]))
    ragged = list(ip.ragged_to_tensor({"r": (None, 3)})([{"r": [[1], [2, 3, 4, 5]]}]))[0]["r"]
    assert ragged.tolist() == [[1, 0, 0], [2, 3, 4]]


def test_batch_training_drops_remainder_and_repeats():
    b = ip.batch(4, is_training=True, repeat=2)
    out = [e["x"].tolist() for e in b(list(_range_source(10)()))]
    assert out == [[0, 1, 2, 3], [4, 5, 6, 7]] * 2
    endless = ip.batch(4, is_training=True)(list(_range_source(5)()))
    assert [next(iter(endless))["x"].tolist() for _ in range(1)] == [[0, 1, 2, 3]]
    with pytest.raises(ValueError):
        ip.batch(4, is_training=True, repeat=0)


def test_batch_eval_pads_last_batch():
    out = list(ip.batch(4, is_training=False)(_range_source(6)()))
    assert [e["x"].tolist() for e in out] == [[0, 1, 2, 3], [4, 5, 0, 0]]
    marked = ip.batch(4, is_training=False, pad_example_fn=lambda ex: {"x": np.int32(-1)})(_range_source(5)())
    assert [e["x"].tolist() for e in marked][-1] == [4, -1, -1, -1]
    strings = list(ip.batch(2, is_training=False)([{"t": "a"}, {"t": "b"}, {"t": "c"}]))
    assert strings[1]["t"].tolist() == ["c", ""]


def test_batch_logical_feeds_validation():
    with pytest.raises(ValueError, match="both"):
        ip.batch(4, is_training=True, global_logical_batch_size=2)
    b = ip.batch(4, is_training=False, global_logical_batch_size=2, logical_feed_indices=[0],
                 pad_example_fn=lambda ex: {"x": np.int32(-1)})
    out = [e["x"].tolist() for e in b(_range_source(4)())]
    assert out == [[0, 1, -1, -1], [2, 3, -1, -1]]


def test_input_module_source_processor_batcher():
    def source(n: int = 6, is_training: bool = False):
        return _range_source(n)

    def double(is_training: bool = False):
        return ip.map_over_dataset(lambda ex: {"x": ex["x"] * (2 if is_training else 1)})

    cfg = ip.Input.default_config().set(
        name="in", is_training=True, source=config_for_function(source).set(n=8),
        processor=config_for_function(double),
        batcher=config_for_function(ip.batch).set(global_batch_size=4, repeat=1))
    inp = cfg.instantiate(parent=None)
    batches = [b["x"].tolist() for b in inp.dataset()]
    assert batches == [[0, 2, 4, 6], [8, 10, 12, 14]]


def test_disable_shuffle_recursively():
    cfg = config_for_function(ip.shuffle).set(shuffle_buffer_size=100)
    outer = config_for_function(ip.chain)
    holder = ip.Input.default_config().set(processor=cfg, source=outer, batcher=outer)
    ip.disable_shuffle_recursively(holder)
    assert holder.processor.shuffle_buffer_size == 0


def _fake_input(values, key="x"):
    from axlearn_b200.common.input_base import Input
    from axlearn_b200.common.config import config_class

    class _Fake(Input):
        @config_class
        class Config(Input.Config):
            is_training: bool = False
            values: list = []

        def dataset(self):
            for v in self._config.values:
                yield {key: v, "train": self._config.is_training}

    return _Fake.default_config().set(values=list(values))


def test_concatenated_and_zip_input():
    cat = ConcatenatedInput.default_config().set(name="c", is_training=True, inputs=[_fake_input([1, 2]), _fake_input([3])])
    out = list(cat.instantiate(parent=None).dataset())
    assert [e["x"] for e in out] == [1, 2, 3] and all(e["train"] for e in out)
    with pytest.raises(ValueError):
        ConcatenatedInput.default_config().set(name="c", is_training=True).instantiate(parent=None)
    z = ZipInput.default_config().set(name="z", is_training=False, inputs={"a": _fake_input([1, 2, 3]), "b": _fake_input([7, 8])})
    out = list(z.instantiate(parent=None).dataset())
    assert [(e["a"]["x"], e["b"]["x"]) for e in out] == [(1, 7), (2, 8)]


@pytest.mark.parametrize("values,ascending,ties,expected", [
    ([2, 2, 4], True, True, [1, 1, 3]),
    ([2, 2, 4], True, False, [1, 2, 3]),
    ([2, 2, 4], False, True, [2, 2, 1]),
    ([2, 2, 4], False, False, [2, 3, 1]),
    ([0.5, 0.1, 0.9, 0.1], True, True, [3, 1, 4, 1]),
    ([], True, True, []),
])
def test_rank_by_value(values, ascending, ties, expected):
    fn = rank_by_value(input_key="v", output_key="r", ascending=ascending, allow_ties=ties)
    out = list(fn([{"v": np.asarray(values, dtype=np.float32)}]))[0]
    assert out["r"].tolist() == expected
    with pytest.raises(NotImplementedError):
        list(fn([{"v": np.zeros((2, 2))}]))


# ------------------------------------------------------------------------------------------ text


def test_text_helpers():
    assert [e["text"] for e in input_text.preprocess_chunks(3)([{"text": "abcdefg"}])] == ["abc", "def", "g"]
    assert list(input_text.strip_accents(["t"])([{"t": "café naïve"}]))[0]["t"] == "cafe naive"
    assert list(input_text.roberta_normalize(cased=False)([{"text": "  Hi There "}]))[0]["text"] == "hi there"
    assert list(input_text.bert_normalize(cased=False)([{"text": "Hello, wörld!\x00 中文"}]))[0]["text"] == "hello , wörld ! 中 文"
    assert list(input_text.join_string_features(["a", "b"], "j")([{"a": "x", "b": "y"}]))[0]["j"] == "x</s>y"
    packed = input_text.pack_strings(["hé", "abc"], 5)
    assert packed.shape == (2, 5) and packed[0, 2] == input_text.STRINGS_BYTE_ARRAY_PAD_VALUE
    assert input_text.unpack_strings(packed) == ["hé", "abc"]
    with pytest.raises(ValueError):
        input_text.pack_strings(["toolong"], 3)
    v = _Vocab()
    ex = list(input_text.tokenize({"text": v}, with_eos=True)([{"text": "a b a"}]))[0]
    assert ex["text"].tolist() == [3, 4, 3, 1] and ex["text_pretokenized"] == "a b a"
    assert input_text.num_bytes(ex["text"], v) == len("a b a") + 1
    tt = list(input_text.add_token_type_ids(["a", "b"])([{"a": np.arange(2), "b": np.arange(3)}]))[0]
    assert tt["token_type_ids"].tolist() == [0, 0, 0, 0, 1, 1, 1, 1]
    assert input_text.infer_bos_id(v) == 2
    chunk = list(input_text.random_chunking(4, seed=0)([{"input_ids": np.arange(10)}]))[0]["input_ids"]
    assert len(chunk) == 4 and (np.diff(chunk) == 1).all()
    assert list(input_text.random_chunking(4)([{"input_ids": np.arange(2)}]))[0]["input_ids"].tolist() == [0, 1]


def test_split_sentences():
    doc = {"text": "Dr. Smith went home. He slept! Did he? Yes.", "id": 7}
    out = list(input_text.split_sentences(passthrough_keys=["id"])([doc]))
    assert [e["text"] for e in out] == ["dr. smith went home.", "he slept!", "did he?", "yes.", ""]
    assert all(e["id"] == 7 for e in out)
    limited = list(input_text.split_sentences(max_sentences_per_example=2)([doc]))
    assert len(limited) == 3 and limited[-1]["text"] == ""


def test_regex_mapped_vocab():
    cls = input_text.with_regex_mapping(_Vocab, encode_mapping=[("\n", " <n> ")], decode_mapping=[(" ?<n> ?", "\n")])
    v = cls()
    assert v.decode(v.encode("a\nb")) == "a\nb"


# ------------------------------------------------------------------------------------------ GLUE


def test_copa_round_trip():
    ex = {"premise": "I packed up.", "question": "cause", "choice1": "hunting", "choice2": "moving", "label": 1}
    pre = list(input_glue.preprocess_copa()([ex]))[0]
    assert pre["premise"] == ["I packed up. What's the CAUSE for this?"] * 2 and pre["choice"] == ["hunting", "moving"]
    other = list(input_glue.preprocess_copa()([{**ex, "question": "effect"}]))[0]
    assert other["premise"][0].endswith("What happened as a RESULT?")
    halves = [{"input_ids": np.arange(4), "target_labels": 1}, {"input_ids": np.arange(4) + 10, "target_labels": 1}]
    post = list(input_glue.postprocess_copa()(halves))[0]
    assert post["input_ids"].shape == (2, 4) and post["target_labels"] == 1
    with pytest.raises(ValueError):
        list(input_glue.postprocess_copa()([halves[0], {**halves[1], "target_labels": 0}]))


def test_roberta_special_tokens():
    v = _Vocab()
    one = list(input_glue.add_special_tokens_for_roberta(v, "a")([{"a": [10, 11]}]))[0]
    assert one["input_ids"].tolist() == [2, 10, 11, 1]
    three = list(input_glue.add_special_tokens_for_roberta(v, ["a", "b", "c"])([{"a": [10], "b": [20], "c": [30]}]))[0]
    assert three["input_ids"].tolist() == [2, 10, 1, 1, 20, 1, 1, 30, 1]


def test_preprocess_record():
    ex = {"passage": "p", "query": "q", "entities": ["c1", "c2"], "answers": ["c1"]}
    out = list(input_glue.preprocess_record()([ex]))[0]
    assert out["passage"] == ["p", "p"] and out["entity"] == ["c1", "c2"] and out["label"].tolist() == [1, 0]


@pytest.mark.parametrize("lens,max_len,expected", [
    ((3, 3), 10, (3, 3)),
    ((10, 2), 8, (6, 2)),
    ((10, 10), 9, (5, 4)),
    ((10, 9, 1), 10, (5, 4, 1)),
    ((7,), 5, (5,)),
])
def test_multi_sequence_truncation(lens, max_len, expected):
    keys = [f"s{i}" for i in range(len(lens))]
    ex = {k: np.arange(n) for k, n in zip(keys, lens)}
    out = list(input_glue.multi_sequence_truncation(max_len, keys)([ex]))[0]
    assert tuple(len(out[k]) for k in keys) == expected
    assert sum(expected) <= max_len
    assert out[keys[0]].tolist() == list(range(expected[0]))      # truncates from the right


def test_add_prefix_concat_sequence_pair():
    qqp = input_glue.add_prefix_concat_sequence_pair(dataset_name="qqp", label_names=["not_duplicate", "duplicate"],
                                                     input_key=("question2", "question1"))
    out = list(qqp([{"question1": "Hello", "question2": "World", "label": 0, "idx": 3},
                    {"question1": "A", "question2": "B", "label": -1, "idx": 4}]))
    assert out[0] == {"source_text": "qqp question1: Hello question2: World", "target_text": "not_duplicate", "idx": 3}
    assert out[1]["target_text"] == "<unk>"
    stsb = input_glue.add_prefix_concat_sequence_pair(dataset_name="stsb", label_names=["none"],
                                                      input_key=("sentence1", "sentence2"))
    assert list(stsb([{"sentence1": "a", "sentence2": "b", "label": 1.77, "idx": 0}]))[0]["target_text"] == "1.8"
    wsc = input_glue.add_prefix_concat_sequence_pair(dataset_name="wsc", label_names=[], input_key="text")
    ex = {"text": "We show an example here .", "span1_text": "example", "span1_index": 3, "span2_text": "We",
          "span2_index": 0, "label": 0, "idx": 1}
    got = list(wsc([ex]))[0]
    assert got["source_text"] == "wsc text: # We # show an * example * here ." and got["target_text"] == "False"
    record = input_glue.add_prefix_concat_sequence_pair(dataset_name="record", label_names=[], input_key="x")
    rex = {"passage": "This is the passage.\n@highlight\nMore", "query": "A @placeholder is a dog.",
           "entities": ["Leopard", "Chihuahua", "Husky"], "answers": ["Chihuahua", "Husky"], "idx": {"passage": 1, "query": 2}}
    got = list(record([rex]))
    assert [g["target_text"] for g in got] == ["Chihuahua", "Husky"]
    assert got[0]["source_text"] == ("record query: A @placeholder is a dog. entities: Leopard, Chihuahua, Husky "
                                     "passage: This is the passage. More")
    assert list(record([{**rex, "answers": []}]))[0]["target_text"] == "<unk>"


_SHARED_VOCAB = _Vocab()


def _make_vocab():
    return _SHARED_VOCAB


def test_text_to_glue_input():
    fn = input_glue.text_to_glue_input(
        is_training=True, input_key=("sentence1", "sentence2"), max_len=12, vocab_cfg=config_for_function(_make_vocab),
        truncation=config_for_function(input_glue.multi_sequence_truncation).set(max_len=8),
        concatenation=config_for_function(input_glue.add_special_tokens_for_roberta),
        normalization=config_for_function(input_text.roberta_normalize).set(cased=False))
    ex = {"sentence1": " A b c d e f ", "sentence2": "g h", "label": 1, "idx": 0}
    out = list(fn([ex]))[0]
    assert set(out) == {"input_ids", "target_labels"} and out["target_labels"] == 1
    ids = out["input_ids"].tolist()
    assert len(ids) == 12 and ids[0] == 2
    # 6 tokens of sentence1 + 2 of sentence2 = 8 within budget; 4 special tokens; no padding left.
    assert ids.count(1) == 3 and 0 not in ids


def test_make_glue_autoregressive_inputs():
    v = _Vocab()
    fn = input_glue.make_glue_autoregressive_inputs(vocab_cfg=v, max_source_length=4, max_target_length=4)
    out = list(fn([{"prefix": [100], "source_ids": [10, 11, 12, 13, 1], "target_labels": [20, 21, 22, 23, 1], "idx": 3}]))[0]
    assert out["source_ids"].tolist() == [10, 11, 12, 1]
    assert out["target_labels"].tolist() == [20, 21, 22, 1]
    assert out["target_ids"].tolist() == [100, 20, 21, 22]
    two = list(fn([{"prefix": [100, 101], "source_ids": [10, 1], "target_labels": [20, 1], "idx": 0}]))[0]
    assert two["target_labels"].tolist() == [-1, 20, 1] and two["target_ids"].tolist() == [100, 101, 20]
