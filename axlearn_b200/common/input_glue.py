"""GLUE / SuperGLUE input processing.

Parity target: axlearn/common/input_glue.py -- ``preprocess_copa`` :34, ``postprocess_copa`` :85,
``add_special_tokens_for_roberta`` :135, ``preprocess_record`` :189,
``multi_sequence_truncation`` :240, ``add_prefix_concat_sequence_pair`` :298 (general, STS-B, WSC
and ReCoRD forms), ``text_to_glue_input`` :596, ``make_glue_autoregressive_inputs`` :683.

Processors map iterables of dict examples to iterables of dict examples (``input_processing``).
"""

from __future__ import annotations

import re
from typing import Any, Iterator, Optional, Sequence, Union

import numpy as np

from axlearn_b200.common.config import InstantiableConfig, maybe_instantiate
from axlearn_b200.common.input_processing import (
    Dataset,
    DatasetToDatasetFn,
    Example,
    chain,
    map_over_dataset,
    rekey,
    trim_and_pad,
)
from axlearn_b200.common.input_text import infer_bos_id, tokenize

SEQ2SEQ_IGNORE_TARGET_LABEL = -1


def _as_keys(key: Union[str, Sequence[str]]) -> list:
    return [key] if isinstance(key, str) else list(key)


def preprocess_copa() -> DatasetToDatasetFn:
    """``{premise, question, choice1, choice2, label}`` -> one element holding BOTH choices
    (lists of 2): the premise extended by the question's template, each choice, the label twice.
    ``unbatch`` downstream, then ``postprocess_copa`` to regroup."""

    def fn(ex: Example) -> Example:
        question = "What's the CAUSE for this?" if ex["question"] == "cause" else "What happened as a RESULT?"
        premise = ex["premise"] + " " + question
        return {"premise": [premise, premise], "choice": [ex["choice1"], ex["choice2"]],
                "label": [ex["label"], ex["label"]]}

    return map_over_dataset(fn)


def postprocess_copa() -> DatasetToDatasetFn:
    """Groups consecutive pairs: ``input_ids [max_len]`` x2 -> ``[2, max_len]``; the pair's labels
    must agree and become one scalar."""

    def process(ds: Dataset) -> Iterator[Example]:
        it = iter(ds)
        for first in it:
            try:
                second = next(it)
            except StopIteration:
                return  # a dangling half pair is dropped, as a batch(2) with remainder dropped would
            if int(first["target_labels"]) != int(second["target_labels"]):
                raise ValueError("Batch has invalid targets.")
            yield {"input_ids": np.stack([np.asarray(first["input_ids"]), np.asarray(second["input_ids"])]),
                   "target_labels": first["target_labels"]}

    return process


def add_special_tokens_for_roberta(vocab_cfg: Any, input_key: Union[str, Sequence[str]], output_key: str = "input_ids",
                                   bos_token: Optional[str] = None) -> DatasetToDatasetFn:
    """``<s> a </s>`` / ``<s> a </s></s> b </s>`` / ...: BOS, the first sequence, EOS, then
    ``EOS seq EOS`` for every further sequence."""
    vocab = maybe_instantiate(vocab_cfg)
    if bos_token:
        bos_id = vocab.piece_to_id(bos_token) if hasattr(vocab, "piece_to_id") else vocab.encode(bos_token)[0]
    else:
        bos_id = infer_bos_id(vocab)
    eos_id = vocab.eos_id
    keys = _as_keys(input_key)
    if not keys:
        raise ValueError("Expected at least one input_key")

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        parts = [[bos_id], ex[keys[0]], [eos_id]]
        for k in keys[1:]:
            parts.extend([[eos_id], ex[k], [eos_id]])
        ex[output_key] = np.concatenate([np.asarray(p, dtype=np.int32) for p in parts])
        return ex

    return map_over_dataset(fn)


def preprocess_record() -> DatasetToDatasetFn:
    """ReCoRD: one element with a row per candidate entity -- the passage and query repeated, the
    entity, and label 1 where the entity is among the answers.  (No entities: one row of passage
    / query with empty entity and label lists, as broadcasting to max(n, 1) gives.)"""

    def fn(ex: Example) -> Example:
        entities = list(ex["entities"])
        answers = set(ex["answers"])
        n = max(len(entities), 1)
        return {"passage": [ex["passage"]] * n, "query": [ex["query"]] * n, "entity": entities,
                "label": np.asarray([int(e in answers) for e in entities], dtype=np.int64)}

    return map_over_dataset(fn)


def multi_sequence_truncation(max_len: int, input_key: Union[str, Sequence[str]] = ()) -> DatasetToDatasetFn:
    """Right-truncates several sequences to ``max_len`` tokens in total.  Every sequence gets
    ``max_len // n``; what the short ones leave unused is split evenly over the long ones, and the
    remainder of that split goes, one token each, to the longest sequences."""
    keys = _as_keys(input_key)
    threshold = max_len // max(1, len(keys))

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        sizes = np.asarray([len(ex[k]) for k in keys], dtype=np.int64)
        thresholds = np.full_like(sizes, threshold)
        total = int(np.minimum(thresholds, sizes).sum())
        truncated = (sizes > thresholds).astype(np.int64)
        n_trunc = max(1, int(truncated.sum()))
        thresholds = thresholds + truncated * ((max_len - total) // n_trunc)
        remainder = (max_len - total) % n_trunc
        # Stable descending order by size: ties keep their original order.
        order = np.argsort(-sizes, kind="stable")[:remainder]
        thresholds[order] += 1
        final = np.minimum(thresholds, sizes)
        for i, k in enumerate(keys):
            ex[k] = ex[k][: int(final[i])]
        return ex

    return map_over_dataset(fn)


def _mark_span(text: str, span_str: str, span_idx: int, mark: str) -> str:
    pattern = r"^((?:\S+\s){" + str(int(span_idx)) + r"})(" + span_str + r")"
    return re.sub(pattern, lambda m: f"{m.group(1)}{mark} {m.group(2)} {mark}", text, count=1)


def add_prefix_concat_sequence_pair(*, dataset_name: str, label_names: Sequence[str],
                                    input_key: Union[str, Sequence[str]] = (), source_key: str = "source_text",
                                    target_key: str = "target_text") -> DatasetToDatasetFn:
    """Text-to-text form: ``source = "<dataset> <key1>: <v1> <key2>: <v2>"`` (keys sorted),
    ``target`` = the label's name (``"<unk>"`` for label -1; STS-B: the score rounded to 0.2 as a
    string; WSC: marks the two spans and targets "True" / "False"; ReCoRD: one example per answer)."""
    keys = sorted(_as_keys(input_key))

    def join_inputs(ex: Example) -> str:
        parts = [dataset_name]
        for k in keys:
            parts += [f"{k}:", ex[k]]
        return " ".join(parts)

    def passthrough(ex: Example, out: Example) -> Example:
        out["idx"] = ex["idx"]
        if "prefix" in ex:
            out["prefix"] = ex["prefix"]
        return out

    def glue_fn(ex: Example) -> Example:
        label = int(ex["label"])
        return passthrough(ex, {source_key: join_inputs(ex), target_key: "<unk>" if label == -1 else label_names[label]})

    def stsb_fn(ex: Example) -> Example:
        score = np.round(float(ex["label"]) * 5) / 5
        return passthrough(ex, {source_key: join_inputs(ex), target_key: f"{score:.1f}"})

    def wsc_fn(ex: Example) -> Example:
        text = _mark_span(ex["text"], re.escape(ex["span1_text"]), ex["span1_index"], "*")
        span2_index = int(ex["span2_index"]) + 2 * int(ex["span1_index"] < ex["span2_index"])
        text = _mark_span(text, re.escape(ex["span2_text"]), span2_index, "#")
        label = int(ex["label"])
        return passthrough(ex, {source_key: " ".join(["wsc", "text:", text]),
                                target_key: "<unk>" if label == -1 else ["False", "True"][label]})

    def record_fn(ds: Dataset) -> Iterator[Example]:
        for ex in ds:
            passage = re.sub(r"(\.|\?|\!|\"|\')\n@highlight\n", r"\1 ", ex["passage"])
            passage = re.sub(r"\n@highlight\n", ". ", passage)
            source = " ".join(["record query:", ex["query"], "entities:", ", ".join(ex["entities"]), "passage:", passage])
            for answer in (list(ex["answers"]) or ["<unk>"]):
                yield passthrough(ex, {source_key: source, target_key: answer})

    if dataset_name == "stsb":
        return map_over_dataset(stsb_fn)
    if dataset_name == "wsc":
        return map_over_dataset(wsc_fn)
    if dataset_name == "record":
        return record_fn
    return map_over_dataset(glue_fn)


def text_to_glue_input(*, is_training: bool, input_key: Union[str, Sequence[str]], max_len: int, vocab_cfg: Any,
                       truncation: InstantiableConfig, concatenation: InstantiableConfig,
                       normalization: Optional[InstantiableConfig] = None) -> DatasetToDatasetFn:
    """normalise -> tokenise every input field (no EOS) -> ``truncation`` (its ``max_len`` leaves
    room for the special tokens) -> ``concatenation`` into "input_ids" -> keep ``input_ids`` and
    ``target_labels`` (= "label") -> pad / trim to ``max_len``."""
    del is_training
    vocab = maybe_instantiate(vocab_cfg)
    keys = _as_keys(input_key)
    if len(keys) < 1:
        raise ValueError("Expected at least one input_key")
    processors: list = []
    if normalization is not None:
        if "input_key" in normalization:
            normalization = normalization.clone(input_key=keys)
        processors.append(normalization)
    processors += [
        tokenize({k: {"vocab": vocab, "add_eos": False} for k in keys}, copy_pretokenized=False),
        truncation.clone(input_key=keys),
        concatenation.clone(vocab_cfg=vocab_cfg, input_key=keys, output_key="input_ids"),
        rekey({"target_labels": "label", "input_ids": "input_ids"}),
        trim_and_pad({"input_ids": max_len}, pad_id=getattr(vocab, "pad_id", 0)),
    ]
    return chain(*processors)


def make_glue_autoregressive_inputs(*, vocab_cfg: Any, max_source_length: int, max_target_length: int) -> DatasetToDatasetFn:
    """Seq2seq (T5-style) GLUE: "source_ids" / "target_labels" arrive with EOS appended; both are
    re-truncated so that they still end in EOS; "target_ids" = prefix + labels shifted; the prefix
    positions (all but its last token) are ignored in "target_labels"."""
    vocab = maybe_instantiate(vocab_cfg)
    eos = np.asarray([vocab.eos_id], dtype=np.int32)

    def fn(ex: Example) -> Example:
        prefix = np.asarray(ex["prefix"], dtype=np.int32)
        source_ids = np.asarray(ex["source_ids"], dtype=np.int32)[:-1]
        target_labels = np.asarray(ex["target_labels"], dtype=np.int32)[:-1]
        source_ids = np.concatenate([source_ids[: max_source_length - 1], eos])
        target_ids = np.concatenate([prefix, target_labels])
        ignored = np.full(max(len(prefix) - 1, 0), SEQ2SEQ_IGNORE_TARGET_LABEL, dtype=np.int32)
        target_labels = np.concatenate([ignored, target_labels])
        target_labels = np.concatenate([target_labels[: max_target_length - 1], eos])
        return dict(idx=ex["idx"], prefix=prefix, source_ids=source_ids, target_ids=target_ids[:max_target_length],
                    target_labels=target_labels)

    return map_over_dataset(fn)
