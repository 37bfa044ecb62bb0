"""Task-specific text preprocessing: masked language modelling and T5 span corruption.

Counterpart of axlearn/common/input_mlm.py (``MLMAction`` :49, ``iid_mlm_actions`` :81,
``roberta_mlm_actions`` :119, ``apply_mlm_mask`` :248, ``text_to_mlm_input`` :560) and
axlearn/common/input_t5.py (``random_spans_noise_mask`` :327, sentinel replacement :415-508,
``make_t5_autoregressive_inputs`` :540).  Functions work on numpy id arrays with an explicit
``numpy.random.Generator`` and are meant for ``Stage.map`` in an input pipeline.
"""

from __future__ import annotations

import enum
from typing import Optional, Sequence

import numpy as np


class MLMAction(enum.IntEnum):
    DO_NOTHING = 0      # not selected
    MASK = 1            # replace by the mask token
    SWAP = 2            # replace by a random token
    KEEP = 3            # selected for prediction but left unchanged


def iid_mlm_actions(length: int, *, rng: np.random.Generator, select_token_prob: float = 0.15,
                    mask_selected_prob: float = 0.8, swap_selected_prob: float = 0.1) -> np.ndarray:
    """Every position is selected independently; a selected position is masked, swapped or kept
    (BERT's 80 / 10 / 10)."""
    if mask_selected_prob + swap_selected_prob > 1:
        raise ValueError("mask and swap probabilities exceed 1")
    selected = rng.random(length) < select_token_prob
    u = rng.random(length)
    action = np.where(u < mask_selected_prob, MLMAction.MASK,
                      np.where(u < mask_selected_prob + swap_selected_prob, MLMAction.SWAP, MLMAction.KEEP))
    return np.where(selected, action, MLMAction.DO_NOTHING).astype(np.int32)


def whole_word_mlm_actions(word_starts: np.ndarray, *, rng: np.random.Generator, select_token_prob: float = 0.15,
                           mask_selected_prob: float = 0.8, swap_selected_prob: float = 0.1) -> np.ndarray:
    """RoBERTa-style: whole words are selected until about ``select_token_prob`` of the tokens are
    covered; all tokens of a word share one action.  ``word_starts [T]`` marks first pieces."""
    length = len(word_starts)
    word_id = np.cumsum(word_starts.astype(np.int64)) - 1
    word_id = np.maximum(word_id, 0)
    num_words = int(word_id.max()) + 1 if length else 0
    budget = max(1, int(round(length * select_token_prob))) if length else 0
    actions = np.full(length, MLMAction.DO_NOTHING, dtype=np.int32)
    covered = 0
    for w in rng.permutation(num_words):
        idx = np.flatnonzero(word_id == w)
        if covered + len(idx) > budget and covered > 0:
            continue
        u = rng.random()
        a = MLMAction.MASK if u < mask_selected_prob else (
            MLMAction.SWAP if u < mask_selected_prob + swap_selected_prob else MLMAction.KEEP)
        actions[idx] = a
        covered += len(idx)
        if covered >= budget:
            break
    return actions


def apply_mlm_mask(input_ids: np.ndarray, actions: np.ndarray, *, mask_id: int, vocab_size: int,
                   rng: np.random.Generator, ignore_target_id: int = 0, special_ids: Sequence[int] = ()) -> dict:
    """``input_ids`` with the actions applied and ``target_labels`` = the original id at selected
    positions, ``ignore_target_id`` elsewhere.  Special tokens (padding, CLS, SEP) are never selected."""
    ids = np.asarray(input_ids)
    actions = np.where(np.isin(ids, list(special_ids)), MLMAction.DO_NOTHING, actions)
    random_ids = rng.integers(0, vocab_size, size=ids.shape)
    out = np.where(actions == MLMAction.MASK, mask_id, np.where(actions == MLMAction.SWAP, random_ids, ids))
    labels = np.where(actions != MLMAction.DO_NOTHING, ids, ignore_target_id)
    return {"input_ids": out.astype(np.int32), "target_labels": labels.astype(np.int32)}


# ------------------------------------------------------------------------------------------
# T5 span corruption.
# ------------------------------------------------------------------------------------------


def _random_segmentation(total: int, num_segments: int, rng: np.random.Generator) -> np.ndarray:
    """``num_segments`` positive integers that add up to ``total``, uniformly over compositions."""
    marks = np.zeros(total - 1, dtype=bool)
    marks[rng.choice(total - 1, num_segments - 1, replace=False)] = True
    starts = np.concatenate([[0], np.flatnonzero(marks) + 1, [total]])
    return np.diff(starts)


def random_spans_noise_mask(length: int, *, rng: np.random.Generator, noise_density: float = 0.15,
                            mean_noise_span_length: float = 3.0) -> np.ndarray:
    """Boolean ``[length]``: alternating non-noise / noise spans, starting with non-noise, with about
    ``noise_density * length`` noise tokens in spans of the given mean length."""
    if length < 2:
        return np.zeros(length, dtype=bool)
    num_noise = int(np.clip(round(length * noise_density), 1, length - 1))
    num_spans = int(max(1, round(num_noise / mean_noise_span_length)))
    num_spans = min(num_spans, num_noise, length - num_noise)
    noise = _random_segmentation(num_noise, num_spans, rng)
    keep = _random_segmentation(length - num_noise, num_spans, rng)
    lengths = np.stack([keep, noise], axis=1).reshape(-1)
    return np.repeat(np.arange(len(lengths)) % 2 == 1, lengths)


def _to_sentinels(ids: np.ndarray, replace: np.ndarray, vocab_size: int) -> np.ndarray:
    """Every maximal run of ``replace`` becomes one sentinel: ``vocab_size - 1`` for the first run,
    ``vocab_size - 2`` for the second, ..."""
    prev = np.concatenate([[False], replace[:-1]])
    first = replace & ~prev
    sentinel = vocab_size - np.cumsum(first)
    out = np.where(first, sentinel, ids)
    return out[~(replace & ~first)]


def apply_t5_mask(input_ids: np.ndarray, *, vocab_size: int, rng: np.random.Generator, noise_density: float = 0.15,
                  mean_noise_span_length: float = 3.0, eos_id: Optional[int] = 1) -> dict:
    """``source_ids``: noise spans replaced by sentinels; ``target_ids``: the sentinels each followed
    by the tokens they replaced (and EOS)."""
    ids = np.asarray(input_ids)
    noise = random_spans_noise_mask(len(ids), rng=rng, noise_density=noise_density,
                                    mean_noise_span_length=mean_noise_span_length)
    source = _to_sentinels(ids, noise, vocab_size)
    target = _to_sentinels(ids, ~noise, vocab_size)
    if eos_id is not None:
        target = np.concatenate([target, [eos_id]])
    return {"source_ids": source.astype(np.int32), "target_ids": target.astype(np.int32)}


def make_t5_autoregressive_inputs(example: dict, *, max_source_len: int, max_target_len: int, bos_id: int = 0,
                                  pad_id: int = 0) -> dict:
    """``source.input_ids``, ``target.input_ids`` (BOS + shifted targets) and ``target_labels``,
    padded or truncated to fixed lengths."""
    def fit(x, n):
        x = np.asarray(x)[:n]
        return np.concatenate([x, np.full(n - len(x), pad_id, dtype=x.dtype)])

    labels = fit(example["target_ids"], max_target_len)
    inputs = np.concatenate([[bos_id], labels[:-1]]).astype(np.int32)
    inputs = np.where(np.concatenate([[True], labels[:-1] != pad_id]), inputs, pad_id)
    return {"source": {"input_ids": fit(example["source_ids"], max_source_len).astype(np.int32)},
            "target": {"input_ids": inputs}, "target_labels": labels.astype(np.int32)}
