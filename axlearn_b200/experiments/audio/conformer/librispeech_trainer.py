"""Conformer speech recognisers on LibriSpeech: ``conformer-test-ctc`` and ``conformer-l-rnnt``.

Counterpart of axlearn/experiments/audio/conformer/{common.py, librispeech_trainer.py}: log-mel
features with SpecAugment and 4x convolutional subsampling, a stack of conformer layers with
Transformer-XL attention (kernel 32 convolutions), and a CTC or RNN-T decoder; Adam (b2 0.98) with
L2 regularisation outside norms / biases / scales, gradient clipping at 1.0, the transformer
learning-rate schedule with 10k warm-up steps, parameter EMA 0.9999; word-error-rate evalers.
Without a dataset directory the inputs are random waveforms.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from axlearn_b200.audio.asr import ASREncoder, ASRModel, CTCDecoderModel, SpeechContextNetwork, SpeechFeatureLayer
from axlearn_b200.audio.conformer import RepeatedConformerLayer
from axlearn_b200.audio.decoder_asr import TransducerDecoderModel
from axlearn_b200.audio.evaler_asr import WordErrorRateMetricCalculator
from axlearn_b200.audio.frontend import LogMelFrontend
from axlearn_b200.audio.spectrum_augmenter import MaskSampler, SpectrumAugmenter
from axlearn_b200.audio.subsamplers import ConvSubSampler
from axlearn_b200.common import checkpointer, evaler, learner, optimizers, schedule
from axlearn_b200.common.config import InstantiableConfig, config_for_class, config_for_function
from axlearn_b200.common.evaler import SpmdEvaler
from axlearn_b200.common.input_fake import FakeSpeechInput
from axlearn_b200.common.layers import set_dropout_rate_recursively
from axlearn_b200.common.param_init import PARAM_REGEXP_WEIGHT, DefaultInitializer, WeightInitializer
from axlearn_b200.common.rnn import LSTMCell
from axlearn_b200.common.trainer import SpmdTrainer

_NUM_FILTERS = 80


def _uniform(scale: float) -> InstantiableConfig:
    return DefaultInitializer.default_config().set(init_by_param_name={
        PARAM_REGEXP_WEIGHT: WeightInitializer.default_config().set(fan=None, distribution="uniform", scale=scale)})


def stack_config(*, num_layers: int, num_heads: int) -> InstantiableConfig:
    cfg = RepeatedConformerLayer.default_config().set(num_layers=num_layers)
    cfg.layer.num_heads = num_heads
    cfg.layer.lconv.conv.window = 32
    return cfg


def feature_config(*, dim: int) -> InstantiableConfig:
    frontend = LogMelFrontend.default_config().set(
        num_filters=_NUM_FILTERS, sample_rate=16000, frame_size_ms=25, hop_size_ms=10, mel_floor=1e-8)
    augmenter = SpectrumAugmenter.default_config().set(
        freq_mask_sampler=MaskSampler.default_config().set(max_num_masks=2, max_mask_length=27),
        time_mask_sampler=MaskSampler.default_config().set(max_num_masks=10, max_mask_length_ratio=0.05))
    return SpeechFeatureLayer.default_config().set(
        output_dim=dim, frontend=frontend, augmenter=augmenter,
        subsampler=ConvSubSampler.default_config().set(norm=None, activation="nn.relu"))


def encoder_config(*, dim: int, feature_dim: int, stack_cfg, dropout_rate: Optional[float] = 0.1) -> InstantiableConfig:
    cfg = ASREncoder.default_config().set(
        dim=dim, feature=feature_config(dim=feature_dim), feature_dim=_NUM_FILTERS // 4 * feature_dim,
        context=SpeechContextNetwork.default_config().set(context=stack_cfg))
    if dropout_rate:
        set_dropout_rate_recursively(cfg.context, dropout_rate)
    return cfg


def rnn_transducer_config(*, vocab_size: int, lm_dim: int, emb_dim: int, joint_dim: int, eos_id: int) -> InstantiableConfig:
    rnn = LSTMCell.default_config().set(max_cell_value=10.0, output_proj=None, param_init=_uniform(0.1))
    rnn.input_proj.bias = True
    cfg = TransducerDecoderModel.default_config().set(vocab_size=vocab_size, lm_dim=lm_dim, joint_dim=joint_dim, eos_id=eos_id)
    cfg.prediction_network.set(emb_dim=emb_dim, rnn_cell=rnn)
    cfg.prediction_network.embedding.param_init = _uniform(1.0)
    return cfg


def ctc_decoder_config(vocab_size: int = 1024) -> InstantiableConfig:
    cfg = CTCDecoderModel.default_config().set(vocab_size=vocab_size)
    cfg.lm_head.param_init = _uniform(0.5)
    return cfg


def adam_learner_config(*, lr_scale: float, warmup_steps: int = 10_000, ema_decay: Optional[float] = 0.9999):
    no_l2 = [".*norm/.*", "(.*/)?bias", "(.*/)?scale", "(.*/)?per_dim_scale/param", "(.*/)?moving_mean",
             "(.*/)?moving_variance"]
    optimizer = config_for_function(optimizers.chain).set(args=[
        config_for_function(optimizers.clip_by_global_norm).set(max_norm=1.0),
        config_for_function(optimizers.adam_optimizer).set(
            learning_rate=config_for_function(schedule.adafactor).set(
                scale=lr_scale, warmup_steps=warmup_steps, decay_power=-0.5, step_offset=1),
            b1=0.9, b2=0.98, eps=1e-9, l2_regularizer_weight=1e-6,
            l2_regularizer_per_param_scale=config_for_function(optimizers.per_param_scale_by_path).set(
                description="l2_regularizer_scale", scale_by_path=[(p, 0) for p in no_l2]))])
    cfg = learner.Learner.default_config().set(optimizer=optimizer)
    if ema_decay:
        cfg.ema.decay = ema_decay
    return cfg


_SIZES = {"test": (4, 4, 1, 2), "s": (512, 144, 16, 4), "m": (512, 256, 16, 4), "l": (512, 512, 17, 8)}


def model_config(*, model_name: str, eos_id: int, vocab_size: int = 1024, dropout_rate: Optional[float] = 0.1):
    """``conformer-{test,s,m,l}-{ctc,rnnt}``."""
    _, size, decoder = model_name.lower().split("-")
    if size not in _SIZES:
        raise ValueError(f"unsupported size {size}")
    feature_dim, encoder_dim, num_layers, num_heads = _SIZES[size]
    if "rnnt" in decoder:
        dec = rnn_transducer_config(vocab_size=vocab_size, lm_dim=640, emb_dim=128, joint_dim=640, eos_id=eos_id)
    elif "ctc" in decoder:
        dec = ctc_decoder_config(vocab_size=vocab_size)
    else:
        raise ValueError(f"unsupported decoder in {model_name}")
    return ASRModel.default_config().set(
        encoder=encoder_config(dim=encoder_dim, feature_dim=feature_dim,
                               stack_cfg=stack_config(num_layers=num_layers, num_heads=num_heads),
                               dropout_rate=dropout_rate),
        decoder=dec.set(input_dim=encoder_dim), dtype=torch.float32)


def _input_fn(*, is_training: bool, split: str, eos_id: int, global_batch_size: int = 2048, vocab_size: int = 1024,
              max_source_len: int = 16000 * 35, max_target_len: int = 512):
    return FakeSpeechInput.default_config().set(
        is_training=is_training, global_batch_size=global_batch_size, eos_id=eos_id, vocab_size=vocab_size,
        max_source_len=max_source_len, max_target_len=max_target_len, seed=sum(map(ord, split)),
        total_num_batches=None if is_training else 2)


class IdVocabulary:
    """Stand-in vocabulary: pieces are the ids themselves (used with the synthetic inputs)."""

    def __init__(self, vocab_size: int = 1024, eos_id: int = 2):
        self.vocab_size, self.eos_id = vocab_size, eos_id

    def decode(self, ids):
        return " ".join(str(i) for i in ids)


def evaler_config_dict(*, input_fn: Callable, max_decode_len: Optional[int] = None, vocab=None) -> dict:
    decode_kwargs = dict(num_decodes=8)
    if max_decode_len:
        decode_kwargs["max_decode_len"] = max_decode_len
    calc = WordErrorRateMetricCalculator.default_config().set(
        model_method="beam_search_decode", vocab=vocab or config_for_class(IdVocabulary), model_method_kwargs=decode_kwargs)
    train_subset = "train_clean100[:512]+train_clean360[:512]+train_other500[:512]"
    out = {}
    for name, kind, split in [("train", "eval", train_subset), ("dev_clean", "eval", "dev_clean"),
                              ("dev_other", "eval", "dev_other"), ("dev_clean", "decoder", "dev_clean"),
                              ("dev_other", "decoder", "dev_other"), ("test_clean", "decoder", "test_clean"),
                              ("test_other", "decoder", "test_other"), ("train", "decoder", train_subset)]:
        cfg = SpmdEvaler.default_config().set(
            input=input_fn(is_training=False, split=split),
            eval_policy=config_for_function(evaler.every_n_steps_policy).set(n=1000, min_step=1), eval_dtype=torch.float32)
        if kind == "decoder":
            cfg.metric_calculator = calc.clone()
        out[f"{kind}_{name}"] = cfg
    return out


def _trainer_config_fn(*, input_cfg, model_cfg, evaler_cfgs: dict, learner_cfg, max_step: int):
    def config_fn():
        cfg = SpmdTrainer.default_config().set(
            name="librispeech_trainer", model=model_cfg.clone(), input=input_cfg.clone(),
            evalers={k: v.clone() for k, v in evaler_cfgs.items()}, learner=learner_cfg.clone(), max_step=max_step,
            train_dtype=None)
        cfg.checkpointer.save_policy = config_for_function(checkpointer.every_n_steps_policy).set(n=100)
        cfg.checkpointer.keep_every_n_steps = 100
        cfg.summary_writer.write_every_n_steps = 200
        return cfg

    return config_fn


def named_trainer_configs() -> dict:
    import functools

    split = "train_clean100+train_clean360+train_other500"
    return {
        "conformer-test-ctc": _trainer_config_fn(
            input_cfg=_input_fn(is_training=True, split=split, eos_id=2, vocab_size=32, global_batch_size=4,
                                max_source_len=8000, max_target_len=8),
            model_cfg=model_config(model_name="conformer-test-ctc", eos_id=2, dropout_rate=None, vocab_size=32),
            evaler_cfgs={}, learner_cfg=adam_learner_config(lr_scale=0.1), max_step=3),
        "conformer-l-rnnt": _trainer_config_fn(
            input_cfg=_input_fn(is_training=True, split=split, eos_id=2),
            model_cfg=model_config(model_name="conformer-l-rnnt", eos_id=2, dropout_rate=0.1),
            evaler_cfgs=evaler_config_dict(input_fn=functools.partial(_input_fn, eos_id=2), max_decode_len=1000),
            learner_cfg=adam_learner_config(lr_scale=0.22097), max_step=500_000),
    }
