"""tokenizers-backed vocabulary on a toy byte-level BPE file with the Llama-3 style specials."""
import pytest

from axlearn_b200.experiments.text.gpt.vocabulary_fuji_v3 import FujiV3Vocabulary


@pytest.fixture(scope="module")
def vocab_file(tmp_path_factory):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, processors, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    specials = ["<|begin_of_text|>", "<|end_of_text|>", "<|finetune_right_pad_id|>"]
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=specials,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog"] * 50 + ["hello world, hello tokens"] * 50, trainer)
    bos = tok.token_to_id("<|begin_of_text|>")
    tok.post_processor = processors.TemplateProcessing(
        single="<|begin_of_text|> $A", special_tokens=[("<|begin_of_text|>", bos)])
    path = tmp_path_factory.mktemp("tok") / "toy.json"
    tok.save(str(path))
    return str(path)


def test_round_trip_and_special_tokens(vocab_file):
    v = FujiV3Vocabulary(vocab_file)
    assert v.bos_id != v.eos_id != v.pad_id and v.vocab_size >= 259
    ids = v.encode("hello world")
    assert ids and ids[0] != v.bos_id and v.eos_id not in ids
    assert v.decode(ids) == "hello world"
    assert v.decode([v.bos_id] + ids + [v.eos_id] + v.encode(" ignored") + [v.pad_id]) == "hello world"
    batch = v.encode_batch(["the lazy dog", "hello tokens"])
    assert batch[0] == v.encode("the lazy dog")
    assert v.decode_batch([batch[0] + [v.pad_id, v.pad_id], batch[1]]) == ["the lazy dog", "hello tokens"]
    pieces = v.tokenizer.encode_as_pieces("hello")
    assert [v.tokenizer.piece_to_id(p) for p in pieces] == v.encode("hello")


def test_works_as_the_lm_input_vocabulary(vocab_file):
    from axlearn_b200.common.input_lm import text_to_lm_training_input

    v = FujiV3Vocabulary(vocab_file)
    rows = list(text_to_lm_training_input([{"text": "the quick brown fox"}, {"text": "hello world"}], vocab=v, max_len=8))
    assert rows and all(len(r["input_ids"]) == 8 for r in rows)
    flat = [t for r in rows for t in r["input_ids"]]
    assert v.eos_id in flat
