"""Tutorial, vision and audio experiment configs: golden hyper-parameters and short runs."""
import os

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.utils import flatten_items

# Hyper-parameters and config names taken from the reference's golden config dumps
# (axlearn/experiments/testdata/<module>/<config>.txt), stored as "key: value" strings.
with open(os.path.join(os.path.dirname(__file__), "testdata", "reference_config_values.json")) as _f:
    _GOLDEN = __import__("json").load(_f)
_REF = "golden"


def _dump(path):
    module, name = path[len(_REF) + 1:-4].split("/")
    return _GOLDEN["values"][f"{module}/{name}"]


def test_logistic_regression_tutorial_trains_to_high_accuracy(tmp_path):
    from axlearn_b200.experiments.logistic_regression import tutorial

    cfg = tutorial.named_trainer_configs()["LogisticRegression"]().set(dir=str(tmp_path), max_step=200)
    assert cfg.learner.optimizer.momentum == 0.9 and cfg.checkpointer.save_policy.n == 200
    trainer = cfg.instantiate(parent=None)
    out = trainer.run(prng.PRNGKey(42))
    assert trainer.step == 200 and float(out["loss"]) < 0.1
    params = dict(flatten_items(trainer.trainer_state["model"]))
    assert set(params) == {"backbone/weight", "backbone/bias"} and params["backbone/weight"].shape == (2, 1)
    assert (params["backbone/weight"] > 0).all()                     # the clusters sit on the diagonal
    assert os.path.isdir(tmp_path / "summaries" / "eval") and os.path.isdir(tmp_path / "checkpoints" / "step_00000200")


@pytest.mark.parametrize("name", ["ResNet-50-ema", "ResNet-18", "ResNet-Testb"])
def test_imagenet_trainer_hyperparameters_match_reference_config_dump(name):
    from axlearn_b200.experiments.vision.resnet import imagenet_trainer

    want = _dump(f"{_REF}/axlearn.experiments.vision.resnet.imagenet_trainer/{name}.txt")
    cfg = imagenet_trainer.named_trainer_configs()[name]()
    assert cfg.max_step == int(want["max_step"])
    assert cfg.checkpointer.save_policy.n == int(want["checkpointer.save_policy.n"])
    assert cfg.checkpointer.keep_every_n_steps == int(want["checkpointer.keep_every_n_steps"])
    lr = cfg.learner.optimizer.learning_rate
    assert lr.peak_lr == pytest.approx(float(want["learner.optimizer.learning_rate.peak_lr"]))
    assert lr.warmup_steps == int(want["learner.optimizer.learning_rate.warmup_steps"])
    assert cfg.learner.optimizer.momentum == float(want["learner.optimizer.momentum"])
    assert cfg.learner.optimizer.weight_decay == float(want["learner.optimizer.weight_decay"])
    assert str(cfg.learner.ema.decay) == want.get("learner.ema.decay", "None")
    assert cfg.model.backbone.hidden_dim == int(want["model.backbone.hidden_dim"])
    blocks = [int(v) for k, v in sorted(want.items()) if k.startswith("model.backbone.num_blocks_per_stage[")]
    assert list(cfg.model.backbone.num_blocks_per_stage) == blocks
    assert cfg.model.num_classes == int(want["model.num_classes"])
    assert set(cfg.evalers) == {k.split("'")[1] for k in want if k.startswith("evalers[")}
    assert set(imagenet_trainer.named_trainer_configs()) == set(
        _GOLDEN["names"]["axlearn.experiments.vision.resnet.imagenet_trainer"])


def test_resnet_test_config_runs_two_steps(tmp_path):
    from axlearn_b200.experiments.vision.resnet import imagenet_trainer

    cfg = imagenet_trainer.named_trainer_configs()["ResNet-Test"]().set(
        dir=str(tmp_path), max_step=2, train_dtype=None, mesh_shape=(1,), mesh_axis_names=("data",))
    cfg.input.image_size = (32, 32)
    cfg.evalers = {}
    trainer = cfg.instantiate(parent=None)
    out = trainer.run(prng.PRNGKey(0))
    assert trainer.step == 2 and torch.isfinite(out["loss"])


def test_librispeech_trainer_matches_reference_config_dump():
    from axlearn_b200.experiments.audio.conformer import librispeech_trainer as lt

    configs = lt.named_trainer_configs()
    assert set(configs) == {"conformer-test-ctc", "conformer-l-rnnt"}
    for name in configs:
        want = _dump(f"{_REF}/axlearn.experiments.audio.conformer.librispeech_trainer/{name}.txt")
        cfg = configs[name]()
        assert cfg.max_step == int(want["max_step"])
        adam = cfg.learner.optimizer.args[1]
        assert adam.learning_rate.scale == pytest.approx(float(want["learner.optimizer.args[1].learning_rate.scale"]))
        assert adam.learning_rate.warmup_steps == int(want["learner.optimizer.args[1].learning_rate.warmup_steps"])
        assert adam.b2 == float(want["learner.optimizer.args[1].b2"]) and adam.eps == float(want["learner.optimizer.args[1].eps"])
        assert adam.l2_regularizer_weight == float(want["learner.optimizer.args[1].l2_regularizer_weight"])
        assert [p for p, _ in adam.l2_regularizer_per_param_scale.scale_by_path] == [
            v.strip("'") for k, v in want.items() if "scale_by_path" in k and k.endswith("[0]")]
        assert cfg.learner.optimizer.args[0].max_norm == float(want["learner.optimizer.args[0].max_norm"])
        assert str(cfg.learner.ema.decay) == want["learner.ema.decay"]
        assert cfg.model.encoder.dim == int(want["model.encoder.dim"])
        assert cfg.model.encoder.context.context.num_layers == int(want["model.encoder.context.context.num_layers"])
        assert cfg.model.encoder.context.context.layer.lconv.conv.window == 32
        assert cfg.checkpointer.save_policy.n == int(want["checkpointer.save_policy.n"])
        assert {k.split("'")[1] for k in want if k.startswith("evalers[")} == set(cfg.evalers)
    rnnt = configs["conformer-l-rnnt"]().model.decoder
    want = _dump(f"{_REF}/axlearn.experiments.audio.conformer.librispeech_trainer/conformer-l-rnnt.txt")
    assert rnnt.lm_dim == int(want["model.decoder.lm_dim"]) and rnnt.joint_dim == int(want["model.decoder.joint_dim"])
    assert rnnt.prediction_network.emb_dim == int(want["model.decoder.prediction_network.emb_dim"])
    assert rnnt.prediction_network.rnn_cell.max_cell_value == float(want["model.decoder.prediction_network.rnn_cell.max_cell_value"])


def test_conformer_test_ctc_runs_its_three_steps(tmp_path):
    from axlearn_b200.experiments.audio.conformer import librispeech_trainer as lt

    cfg = lt.named_trainer_configs()["conformer-test-ctc"]().set(
        dir=str(tmp_path), mesh_shape=(1,), mesh_axis_names=("data",))
    trainer = cfg.instantiate(parent=None)
    out = trainer.run(prng.PRNGKey(0))
    assert trainer.step == 3 and torch.isfinite(out["loss"])


def test_word_error_counts():
    from axlearn_b200.audio.evaler_asr import compute_word_errors, word_errors

    assert word_errors("a b c".split(), "a b c".split()) == dict(substitutions=0, deletions=0, insertions=0)
    assert word_errors("a x c d".split(), "a b c".split()) == dict(substitutions=1, deletions=0, insertions=1)
    assert word_errors("a".split(), "a b c".split()) == dict(substitutions=0, deletions=2, insertions=0)
    total = compute_word_errors(["the cat sat", "", "x"], ["the cat sat down", "hello world", ""])
    assert total == dict(num_words=6, substitutions=0, deletions=3, insertions=0, num_examples=2)


def test_word_error_rate_calculator_sums_over_batches():
    from axlearn_b200.audio.decoder_asr import DecodeOutputs
    from axlearn_b200.audio.evaler_asr import WordErrorRateMetricCalculator
    from axlearn_b200.common.base_model import BaseModel
    from axlearn_b200.common.config import config_for_class
    from axlearn_b200.experiments.audio.conformer.librispeech_trainer import IdVocabulary

    class Echo(BaseModel):
        """Decodes to the labels with the first token replaced: one substitution per utterance."""

        def beam_search_decode(self, input_batch, num_decodes):
            seq = input_batch["target_labels"].clone()
            seq[:, 0] = 999
            pad = (seq < 0) | (seq == 2)
            return DecodeOutputs(raw_sequences=seq[:, None], sequences=seq[:, None], paddings=pad[:, None],
                                 scores=torch.zeros(seq.shape[0], 1))

    model = Echo.default_config().set(name="m").instantiate(parent=None)
    calc = WordErrorRateMetricCalculator.default_config().set(
        name="wer", vocab=config_for_class(IdVocabulary), model_method_kwargs=dict(num_decodes=1)).instantiate(
        parent=None, model=model, model_param_partition_specs={})
    state = calc.init_state(prng_key=prng.PRNGKey(0), model_params={})
    outs = []
    for labels in (torch.tensor([[5, 6, 7, 2, -1], [8, 9, 2, -1, -1]]), torch.tensor([[4, 2, -1, -1, -1]])):
        r = calc.forward({"target_labels": labels}, model_params={}, state=state)
        state = r["state"]
        outs.append(r["output"])
    summaries = calc.get_summaries(model_params={}, state=state, all_forward_outputs=outs)
    assert float(summaries["word_errors/wer"].mean) == pytest.approx(3 / 6)
    assert float(summaries["word_errors/substitutions"].mean) == pytest.approx(0.5)
    assert float(summaries["word_errors/num_examples"].mean) == 3


def test_pajama_and_deterministic_trainer_names_are_the_reference_sets():
    from axlearn_b200.experiments.text.gpt import deterministic_trainer, pajama_trainer

    def names(module):
        return set(_GOLDEN["names"][f"axlearn.experiments.text.gpt.{module}"])

    assert set(pajama_trainer.named_trainer_configs()) == names("pajama_trainer")
    assert set(deterministic_trainer.named_trainer_configs()) == names("deterministic_trainer")
    want = _dump(f"{_REF}/axlearn.experiments.text.gpt.pajama_trainer/gala-1B-flash-sp-rp.txt")
    cfg = pajama_trainer.named_trainer_configs()["gala-1B-flash-sp-rp"]()
    assert cfg.max_step == int(want["max_step"])
    weights = [float(v) for k, v in want.items() if k.endswith("['weight']") and "data_mixture_components" in k]
    assert [c.weight for c in cfg.input.source.data_mixture_components] == weights
    assert cfg.input.global_batch_size == int(want["input.input_dispatcher.global_logical_batch_size"])
    assert set(cfg.evalers) == {k.split("'")[1] for k in want if k.startswith("evalers[")}
    det = deterministic_trainer.named_trainer_configs()["honeycrisp-test-flash-pajama-15t-49k"]()
    assert det.save_input_iterator is True


def test_pajama_test_config_trains_on_the_synthetic_mixture_and_resumes_its_input(tmp_path):
    from axlearn_b200.common.utils import set_data_dir
    from axlearn_b200.experiments.text.gpt import pajama_trainer

    with set_data_dir("FAKE"):
        cfg = pajama_trainer.named_trainer_configs()["gala-test-sp-rp"]().set(
            dir=str(tmp_path), max_step=3, mesh_shape=(1,), mesh_axis_names=("data",), save_input_iterator=True)
        cfg.model.decoder.vocab_size = 259                   # the byte vocabulary stands in for sentencepiece
        cfg.evalers = {}
        cfg.input.prefetch = 0
        trainer = cfg.instantiate(parent=None)
        out = trainer.run(prng.PRNGKey(0))
        assert trainer.step == 3 and torch.isfinite(out["loss"])
        batch = next(iter(trainer.input.dataset()))
        assert batch["input_ids"].shape == (16, 64) and batch["input_ids"].max() < 259
