"""Trainer configs over pre-tokenised, pre-batched corpora, for bit-reproducible runs.

Counterpart of axlearn/experiments/text/gpt/deterministic_trainer.py: the training set is already
tokenised and packed in a fixed order (a flat token file, read in order without shuffling), the
input iterator is checkpointed with the model, and only flash-attention configs are generated:
``<model>-flash-<dataset>`` for ``pajama-2t-32k`` (Gala) and ``pajama-15t-49k`` (Honeycrisp).
"""

from __future__ import annotations

import os
from typing import Callable

import numpy as np

from axlearn_b200.common import input_pipeline as ip
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.utils import get_data_dir
from axlearn_b200.experiments.text.gpt import gala, honeycrisp
from axlearn_b200.experiments.text.gpt.pajama_trainer import eval_input_sources

_TRAINING_DATASETS = {
    "pajama-2t-32k": dict(dataset_name="pajama_2t_32k_deterministic:1.0.0", vocab_size=32 * 1024,
                          max_sequence_length=4096, model_versions=(gala,)),
    "pajama-15t-49k": dict(dataset_name="pajama_15t_49k_deterministic:1.0.0", vocab_size=48 * 1024,
                           max_sequence_length=4096, model_versions=(honeycrisp,)),
}


def pretokenized_source(*, dataset_name: str, max_sequence_length: int, vocab_size: int):
    """``<data_dir>/<dataset>/train.bin`` (uint16 or uint32 token ids) read window by window in file
    order, sharded by position; synthetic tokens without a data directory."""

    def build(shard_index: int, shard_count: int) -> ip.Stage:
        data_dir = get_data_dir()
        if data_dir in (None, "FAKE"):
            rng = np.random.default_rng(0)
            n = 64
            tokens = rng.integers(1, min(vocab_size, 30000), size=(n, max_sequence_length + 1)).astype(np.int32)
            source: ip.Source = ip.ListSource([{"input_ids": t[:-1], "target_labels": t[1:]} for t in tokens])
        else:
            path = os.path.join(data_dir, dataset_name.replace(":", "_"), "train.bin")
            source = ip.TokenFileSource(path, length=max_sequence_length,
                                        dtype="uint16" if vocab_size <= 65536 else "uint32")
        return ip.read(source, shuffle=False, num_epochs=None, shard_index=shard_index, shard_count=shard_count)

    return build


def _train_input_source_fn(*, dataset_name: str, **info) -> Callable:
    def fn(vocab_size: int, max_sequence_length: int):
        if vocab_size != info["vocab_size"]:
            raise ValueError(f"vocab_size mismatch for {dataset_name}: {vocab_size} vs. {info['vocab_size']}")
        if max_sequence_length > info["max_sequence_length"]:
            raise ValueError(f"max_sequence_length mismatch for {dataset_name}: {max_sequence_length} vs. {info}")
        return config_for_function(pretokenized_source).set(
            dataset_name=dataset_name, max_sequence_length=max_sequence_length, vocab_size=vocab_size)

    return fn


def _save_input_iterator(fn):
    def wrapped():
        return fn().set(save_input_iterator=True)

    return wrapped


def named_trainer_configs() -> dict:
    configs = {}
    for training_dataset_name, info in _TRAINING_DATASETS.items():
        info = dict(info)
        for module in info.pop("model_versions"):
            for name, fn in module.trainer_configs(_train_input_source_fn(**info), eval_input_sources).items():
                if "flash" in name:
                    configs[f"{name}-{training_dataset_name}"] = _save_input_iterator(fn)
    return configs
