"""Text input plumbing shared by the LM experiments: vocabularies and dataset mixtures.

Counterpart of axlearn/experiments/text/common.py (``DataMixtureComponent``, ``vocab`` :62,
``tfds_text_source`` :20) and of ``mixture_train_input_source`` in
axlearn/experiments/text/gpt/common.py.  Datasets are directories of JSON-lines shards
``<data_dir>/<name with ':' and '/' as '_'>/<split>*.jsonl`` with a ``text`` field; with the data
directory ``FAKE`` (or none) every component is a synthetic corpus.
"""

from __future__ import annotations

import dataclasses
import glob
import os
import re
from typing import Callable, Optional, Sequence

import numpy as np

from axlearn_b200.common import input_pipeline as ip
from axlearn_b200.common.config import InstantiableConfig, config_for_class, maybe_instantiate
from axlearn_b200.common.input_lm import ByteVocabulary, SentencePieceVocabulary, text_to_lm_training_input
from axlearn_b200.common.utils import get_data_dir


@dataclasses.dataclass
class DataMixtureComponent:
    name: str
    weight: float
    shuffle_buffer_size: int = 0
    split: str = "train"
    info: str = ""


def vocab(*, sentencepiece_model_name: str, num_extra_ids: Optional[int] = None):
    """The sentencepiece model ``<data_dir>/tokenizers/sentencepiece/<name>``; without a data
    directory (or when the file is absent) a byte-level vocabulary."""
    del num_extra_ids
    data_dir = get_data_dir()
    if data_dir not in (None, "FAKE"):
        path = os.path.join(data_dir, "tokenizers", "sentencepiece", sentencepiece_model_name)
        if os.path.exists(path):
            return SentencePieceVocabulary.default_config().set(sentencepiece_model_file=path).instantiate()
    return ByteVocabulary.default_config().instantiate()


def _fake_documents(seed: int, n: int = 256) -> list[dict]:
    rng = np.random.default_rng(seed)
    words = ["lorem", "ipsum", "dolor", "sit", "amet", "consectetur", "adipiscing", "elit", "sed", "do"]
    return [{"text": " ".join(rng.choice(words, size=int(rng.integers(5, 60))))} for _ in range(n)]


def text_source(*, dataset_name: str, split: str, is_training: bool, seed: int = 0) -> Callable[[int, int], ip.Stage]:
    """``(shard_index, shard_count) -> Stage`` of ``{"text"}`` documents."""

    def build(shard_index: int, shard_count: int) -> ip.Stage:
        data_dir = get_data_dir()
        if data_dir in (None, "FAKE"):
            source: ip.Source = ip.ListSource(_fake_documents(seed + sum(map(ord, dataset_name))))
        else:
            pattern = os.path.join(data_dir, re.sub(r"[:/]", "_", dataset_name), f"{split.split('[')[0]}*.jsonl")
            files = sorted(glob.glob(pattern))
            if not files:
                raise FileNotFoundError(f"no shards match {pattern}")
            source = ip.JsonLinesSource(files)
        return ip.read(source, shuffle=is_training, seed=seed, num_epochs=None if is_training else 1,
                       shard_index=shard_index, shard_count=shard_count)

    return build


class _Tokenize(ip.Stage):
    """Documents -> fixed-length LM examples through ``text_to_lm_training_input``; restorable at
    the boundaries of its document windows."""

    def __init__(self, parent: ip.Stage, *, vocab, max_len: int, window_size: int, **kwargs):
        self._parent, self._vocab, self._max_len, self._window, self._kw = parent, vocab, max_len, window_size, kwargs
        self._ready: list = []
        self._i = 0
        self._at_window = parent.state()

    def __next__(self):
        while self._i >= len(self._ready):
            self._at_window = self._parent.state()
            docs = []
            for _ in range(self._window):
                try:
                    docs.append(next(self._parent))
                except StopIteration:
                    break
            if not docs:
                raise StopIteration
            self._ready = [
                {k: np.asarray(v, dtype=np.int32) for k, v in ex.items()}
                for ex in text_to_lm_training_input(docs, vocab=self._vocab, max_len=self._max_len,
                                                    window_size=self._window, **self._kw)]
            self._i = 0
        self._i += 1
        return self._ready[self._i - 1]

    def state(self):
        return {"parent": self._at_window, "emitted": self._i}

    def set_state(self, state):
        self._parent.set_state(state["parent"])
        self._ready, self._i = [], 0
        if state["emitted"]:
            next(self)
            self._i = int(state["emitted"])


def lm_text_preprocessor(*, vocab_cfg, max_sequence_length: int, replace_newlines_with: str = "\\n",
                         window_size: int = 128, max_padding_fraction: float = 1.0, shuffle_buffer_size: int = 0):
    """``Stage of documents -> Stage of LM examples``."""

    def fn(ds: ip.Stage) -> ip.Stage:
        return _Tokenize(ds, vocab=maybe_instantiate(vocab_cfg), max_len=max_sequence_length, window_size=window_size,
                         replace_newlines_with=replace_newlines_with, max_padding_fraction=max_padding_fraction,
                         shuffle_buffer_size=shuffle_buffer_size)

    return fn


def mixture_train_input_source(*, data_mixture_components: Sequence[DataMixtureComponent], vocab_cfg,
                               max_sequence_length: int, preprocessor=None, replace_newlines_with: str = "\\n",
                               seed: int = 0) -> Callable[[int, int], ip.Stage]:
    """Every component is tokenised and packed on its own, then examples are drawn from the
    components with probability proportional to their weights."""
    pre_cfg = preprocessor

    def build(shard_index: int, shard_count: int) -> ip.Stage:
        streams, weights = [], []
        for k, comp in enumerate(data_mixture_components):
            docs = text_source(dataset_name=comp.name, split=comp.split, is_training=True, seed=seed + k)(
                shard_index, shard_count)
            if pre_cfg is not None:
                cfg = pre_cfg.clone(vocab_cfg=vocab_cfg, max_sequence_length=max_sequence_length,
                                    replace_newlines_with=replace_newlines_with)
                pre = cfg.instantiate()
            else:
                pre = lm_text_preprocessor(vocab_cfg=vocab_cfg, max_sequence_length=max_sequence_length,
                                           replace_newlines_with=replace_newlines_with)
            streams.append(pre(docs))
            weights.append(comp.weight)
        return ip.sample_from_datasets(streams, weights, seed=seed)

    return build
