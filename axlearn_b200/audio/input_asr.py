"""Input processing for speech recognition (reference: axlearn/audio/input_asr.py:15-205).

Processors over plain iterables of ``dict`` examples (``common/input_processing.py``):

* ``speech_input``: optional scaling, filtering of empty / over-long audio, padding or truncation
  to ``max_len`` samples; emits ``inputs`` (float32) and ``paddings`` (True at padding positions);
* ``text_input``: tokenises the transcript into ``target_labels``, filters by length, appends EOS
  *before* truncation and pads with -1 (an out-of-vocabulary id, so that losses skip it);
* ``make_autoregressive_inputs``: ``input_ids`` = BOS followed by ``target_labels`` shifted right;
* ``pad_example_fn``: the padding example for evaluation batches (all-padding source, -1 tokens).
"""

from __future__ import annotations

from typing import Any, Optional

import numpy as np

from axlearn_b200.common import input_processing as ipx
from axlearn_b200.common import input_text
from axlearn_b200.common.config import maybe_instantiate


def _filter_by_length(*, input_key: str, min_len: Optional[int] = None,
                      max_len: Optional[int] = None) -> ipx.DatasetToDatasetFn:
    """Keeps examples whose ``shape[-1]`` lies in ``[min_len, max_len]``."""

    def keep(ex: ipx.Example) -> bool:
        n = np.shape(ex[input_key])[-1]
        return (min_len is None or min_len <= n) and (max_len is None or n <= max_len)

    return ipx.filter_examples(keep)


def _normalize_by_scale(*, input_key: str, scale: float) -> ipx.DatasetToDatasetFn:
    if scale <= 0:
        raise ValueError(f"scale must be strictly positive, got {scale}.")

    def fn(ex: ipx.Example) -> ipx.Example:
        ex = dict(ex)
        ex[input_key] = np.asarray(ex[input_key], dtype=np.float32) / scale
        return ex

    return ipx.map_over_dataset(fn)


def speech_input(*, max_len: int, input_key: str = "speech", normalize_by_scale: Optional[float] = None,
                 truncate: bool = False) -> ipx.DatasetToDatasetFn:
    """``{input_key: [audio_len], ...}`` -> ``{"inputs": float32 [max_len], "paddings": bool [max_len],
    ...}``; examples longer than ``max_len`` are dropped unless ``truncate``."""
    if max_len < 1:
        raise ValueError("Max length must be at least 1.")

    def to_fixed_length(ex: ipx.Example) -> ipx.Example:
        ex = dict(ex)
        audio = np.asarray(ex.pop(input_key))
        length = audio.shape[-1]
        ex["inputs"] = ipx.trim_and_pad_tensor(audio, max_len=max_len).astype(np.float32)
        ex["paddings"] = np.arange(max_len) >= length
        return ex

    processors = []
    if normalize_by_scale:
        processors.append(_normalize_by_scale(input_key=input_key, scale=normalize_by_scale))
    processors.append(_filter_by_length(input_key=input_key, min_len=1, max_len=None if truncate else max_len))
    return ipx.chain(*processors, ipx.map_over_dataset(to_fixed_length))


def text_input(*, max_len: int, vocab: Any, input_key: str = "text", truncate: bool, min_len: int = 1,
               eos_id: Optional[int] = None) -> ipx.DatasetToDatasetFn:
    """Adds ``target_labels`` ([max_len] int32, -1 padded, EOS appended unless truncated away); all
    other keys pass through.  Without ``truncate`` an example whose labels plus EOS exceed
    ``max_len`` is dropped."""
    if max_len < 1:
        raise ValueError("Max length must be at least 1.")
    spm_vocab = maybe_instantiate(vocab)
    if eos_id is None:
        eos_id = spm_vocab.eos_id
    pad_id = -1

    def trim_and_pad_with_eos(ex: ipx.Example) -> ipx.Example:
        ex = dict(ex)
        labels = np.concatenate([np.asarray(ex["target_labels"], dtype=np.int32), np.asarray([eos_id], dtype=np.int32)])
        ex["target_labels"] = ipx.trim_and_pad_tensor(labels, max_len=max_len, pad_id=pad_id)
        return ex

    processors = [
        ipx.rekey({"target_labels": input_key}, retain_original_inputs=True),
        input_text.tokenize({"target_labels": spm_vocab}, copy_pretokenized=False),
        _filter_by_length(input_key="target_labels", min_len=min_len),
    ]
    if not truncate:
        processors.append(_filter_by_length(input_key="target_labels", max_len=max_len - 1))
    return ipx.chain(*processors, ipx.map_over_dataset(trim_and_pad_with_eos))


def make_autoregressive_inputs(*, vocab: Any, bos_id: Optional[int]) -> ipx.DatasetToDatasetFn:
    """``input_ids = [bos_id] + target_labels[:-1]``; ``bos_id=None`` uses ``vocab_size`` (an id just
    past the vocabulary, for models whose embedding reserves it)."""
    spm_vocab = maybe_instantiate(vocab)
    bos = spm_vocab.vocab_size if bos_id is None else bos_id

    def fn(ex: ipx.Example) -> ipx.Example:
        ex = dict(ex)
        labels = np.asarray(ex["target_labels"])
        ex["input_ids"] = np.concatenate([np.asarray([bos], dtype=labels.dtype), labels[:-1]])
        return ex

    return ipx.map_over_dataset(fn)


def pad_example_fn(example: ipx.Example) -> ipx.Example:
    """Padding example for ``{"source": {"inputs", "paddings"}, "target": {"input_ids"},
    "target_labels"}`` batches: the source is all padding and every token is -1."""
    out = ipx.default_pad_example_fn(example)
    out["source"]["paddings"] = np.ones_like(np.asarray(out["source"]["paddings"]), dtype=bool)
    out["target"]["input_ids"] = np.full_like(np.asarray(out["target"]["input_ids"]), -1, dtype=np.int32)
    out["target_labels"] = np.full_like(np.asarray(out["target_labels"]), -1, dtype=np.int32)
    return out
