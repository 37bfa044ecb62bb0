"""Gala and Honeycrisp on the SlimPajama / RedPajama mixture: ``<model>-sp-rp`` trainer configs.

Counterpart of axlearn/experiments/text/gpt/pajama_trainer.py:40-174: seven weighted corpora
(common crawl 0.726, C4 0.081, GitHub 0.049, books 0.021, arXiv 0.023, Wikipedia 0.05,
StackExchange 0.05), each shuffled and packed on its own before mixing; evaluation on a slice of
OpenWebText2.
"""

from __future__ import annotations

from typing import Callable

from axlearn_b200.common import input_pipeline as ip
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.utils import get_data_dir
from axlearn_b200.experiments.text.common import (
    DataMixtureComponent,
    lm_text_preprocessor,
    mixture_train_input_source,
    text_source,
    vocab,
)
from axlearn_b200.experiments.text.gpt import gala, honeycrisp

_SENTENCEPIECE_MODEL_NAME = {32 * 1024: "bpe_32k_c4.model", 48 * 1024: "bpe_48k_honeycrisp.model"}
_SHUFFLE_BUFFER_SIZE = 8192
REPLACE_NEWLINES_WITH = "<n>"

DATASETS = {
    "sp-rp": [
        DataMixtureComponent(name="rpg/common_crawl:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.726),
        DataMixtureComponent(name="slimpajama/c4:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.081),
        DataMixtureComponent(name="slimpajama/github:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.049),
        DataMixtureComponent(name="slimpajama/book:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.021),
        DataMixtureComponent(name="slimpajama/arxiv:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.023),
        DataMixtureComponent(name="slimpajama/wikipedia:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.05),
        DataMixtureComponent(name="slimpajama/stackexchange:1.0.0", split="train", shuffle_buffer_size=_SHUFFLE_BUFFER_SIZE, weight=0.05),
    ]
}


def _vocab_cfg(vocab_size: int):
    return config_for_function(vocab).set(sentencepiece_model_name=_SENTENCEPIECE_MODEL_NAME.get(vocab_size, "bpe_32k_c4.model"))


def _eval_source(*, dataset_name: str, split: str, vocab_cfg, max_sequence_length: int):
    def build(shard_index: int, shard_count: int) -> ip.Stage:
        docs = text_source(dataset_name=dataset_name, split=split, is_training=False)(shard_index, shard_count)
        return lm_text_preprocessor(vocab_cfg=vocab_cfg, max_sequence_length=max_sequence_length,
                                    replace_newlines_with=REPLACE_NEWLINES_WITH)(docs)

    return build


def eval_input_sources(*, vocab_size: int, max_sequence_length: int) -> dict:
    """``{evaler name: input source config}``."""
    return {
        name: config_for_function(_eval_source).set(
            dataset_name=dataset_name, split=split, vocab_cfg=_vocab_cfg(vocab_size),
            max_sequence_length=max_sequence_length)
        for dataset_name, name, split in (("pile/openwebtext_2:1.0.0", "openwebtext_2", "test[:5000]"),)
    }


def train_input_source_fn(*, train_data_mixture_components) -> Callable:
    """``(vocab_size, max_sequence_length) -> input source config`` over the mixture."""

    def fn(vocab_size: int, max_sequence_length: int):
        pre = config_for_function(lm_text_preprocessor).set(
            max_padding_fraction=0.5, shuffle_buffer_size=0 if get_data_dir() in (None, "FAKE") else _SHUFFLE_BUFFER_SIZE)
        return config_for_function(mixture_train_input_source).set(
            data_mixture_components=train_data_mixture_components, vocab_cfg=_vocab_cfg(vocab_size),
            max_sequence_length=max_sequence_length, preprocessor=pre, replace_newlines_with=REPLACE_NEWLINES_WITH)

    return fn


def named_trainer_configs() -> dict:
    configs = {}
    for module in (gala, honeycrisp):
        for dataset_name, components in DATASETS.items():
            source = train_input_source_fn(train_data_mixture_components=components)
            for name, fn in module.trainer_configs(source, eval_input_sources).items():
                configs[f"{name}-{dataset_name}"] = fn
    return configs
