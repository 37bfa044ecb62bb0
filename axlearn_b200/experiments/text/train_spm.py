"""Trains a SentencePiece model on a text corpus (reference: axlearn/experiments/text/train_spm.py).

    python -m axlearn_b200.experiments.text.train_spm \\
        --input 'corpus/*.jsonl' --spm_config_file bpe_32k.json --model_name c4 \\
        --max_train_examples 100000 --output_dir tokenizers/sentencepiece

The reference reads a TFDS dataset; here the corpus is any mix of ``.jsonl`` files (one object per
line), ``.tfrecord`` files of ``tf.train.Example`` and plain text files (one sentence per line),
read through the framework's own sources.  Everything else follows the reference: the JSON config
file is passed to the trainer as keyword arguments over a small set of defaults; ``pad_id`` (and
only ``pad_id``) must be 0 so that the ids agree with padded batches; the model is named
``spm_{config}_{model_name}``; a few held-out sentences are encoded and decoded as a check; the
``.model`` / ``.vocab`` files are copied to the output directory.

SentencePiece training runs on the CPU and keeps the corpus in memory.
"""

from __future__ import annotations

import argparse
import glob
import json
import logging
import multiprocessing
import os
import random
import re
import shutil
from typing import Any, Iterator, Optional, Sequence


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__.split("\n", 1)[0])
    ap.add_argument("--input", nargs="+", required=True, help="Corpus files or globs (.jsonl, .tfrecord, text).")
    ap.add_argument("--text_key", default="text", help="Field that holds the text in structured inputs.")
    ap.add_argument("--max_train_examples", type=int, default=100_000_000)
    ap.add_argument("--shuffle_buffer_size", type=int, default=64 * 1024)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--spm_config_file", required=True,
                    help="JSON file whose key / value pairs go to the SentencePiece trainer.")
    ap.add_argument("--model_name", default=None)
    ap.add_argument("--output_dir", default=None, help="Default: ./tokenizers/sentencepiece")
    ap.add_argument("--num_eval_examples", type=int, default=10)
    return ap


def expand_inputs(patterns: Sequence[str]) -> list[str]:
    paths: list[str] = []
    for p in patterns:
        matched = sorted(glob.glob(p))
        if not matched:
            raise FileNotFoundError(p)
        paths += matched
    return paths


def iter_texts(paths: Sequence[str], *, text_key: str = "text") -> Iterator[str]:
    """Non-empty texts of the corpus, in file order."""
    from axlearn_b200.common import tfrecord

    for path in paths:
        if path.endswith((".jsonl", ".json")):
            with open(path, encoding="utf-8") as f:
                for line in f:
                    if line.strip():
                        text = json.loads(line)[text_key]
                        if text:
                            yield text
        elif path.endswith((".tfrecord", ".tfrecords")) or ".tfrecord-" in os.path.basename(path):
            for record in tfrecord.read_tfrecords(path, check_crc=False):
                values = tfrecord.decode_example(record).get(text_key) or []
                if len(values) and values[0]:
                    yield values[0].decode("utf-8")
        else:
            with open(path, encoding="utf-8") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if line:
                        yield line


def shuffled(it: Iterator[str], *, buffer_size: int, seed: int) -> Iterator[str]:
    """Streaming shuffle with a bounded buffer (what ``train_shuffle_buffer_size`` does upstream)."""
    if buffer_size <= 1:
        yield from it
        return
    rng, buf = random.Random(seed), []
    for x in it:
        if len(buf) < buffer_size:
            buf.append(x)
            continue
        j = rng.randrange(buffer_size)
        yield buf[j]
        buf[j] = x
    rng.shuffle(buf)
    yield from buf


def build_spm_config(model_prefix: str, *, spm_config_file: str, max_train_examples: int) -> dict[str, Any]:
    configs: dict[str, Any] = dict(
        model_prefix=model_prefix,
        character_coverage=1,
        model_type="unigram",
        num_threads=min(multiprocessing.cpu_count(), 128),
        input_sentence_size=max_train_examples,
        train_extremely_large_corpus=True,
        shuffle_input_sentence=True,
        max_sentence_length=4192,
    )
    with open(spm_config_file, encoding="utf-8") as f:
        configs.update(json.load(f))
    unk_id, bos_id, eos_id = configs.get("unk_id"), configs.get("bos_id"), configs.get("eos_id")
    if configs.get("pad_id", 0) != 0 or 0 in (unk_id, bos_id, eos_id):
        raise ValueError("pad_id (and only pad_id) must be 0: padded batches use id 0 for padding.")
    return configs


def format_name(config_name: str, model_name: Optional[str] = None) -> str:
    config_name = os.path.splitext(os.path.basename(config_name))[0]
    config_name = f"{config_name}_{model_name}" if model_name else config_name
    return re.sub("[:/.]", "_", f"spm_{config_name}")


def train(args: argparse.Namespace) -> str:
    """Trains, validates and copies the model; returns the path of the ``.model`` file."""
    import itertools

    import sentencepiece as spm

    paths = expand_inputs(args.input)
    output_dir = args.output_dir or os.path.join("tokenizers", "sentencepiece")
    os.makedirs(output_dir, exist_ok=True)
    model_name = format_name(args.spm_config_file, args.model_name)
    # Train into the output directory's own scratch name so that a relative model prefix does not
    # litter the caller's working directory.
    work_prefix = os.path.join(output_dir, f".{model_name}.work")
    cfg = build_spm_config(work_prefix, spm_config_file=args.spm_config_file,
                           max_train_examples=args.max_train_examples)
    sentences = itertools.islice(
        shuffled(iter_texts(paths, text_key=args.text_key), buffer_size=args.shuffle_buffer_size, seed=args.seed),
        args.max_train_examples)
    spm.SentencePieceTrainer.train(sentence_iterator=sentences, **cfg)  # pylint: disable=no-member

    outputs = []
    for ext in (".model", ".vocab"):
        src = work_prefix + ext
        if os.path.exists(src):
            dst = os.path.join(output_dir, model_name + ext)
            shutil.move(src, dst)
            outputs.append(dst)
    model_file = os.path.join(output_dir, model_name + ".model")
    logging.info("Model output to: %s", model_file)

    sp = spm.SentencePieceProcessor(model_file=model_file)
    for i, query in enumerate(itertools.islice(iter_texts(paths, text_key=args.text_key), args.num_eval_examples)):
        ids = sp.encode(query)
        logging.info("== Eval case: %d ==\nQuery: %s\nEncoded IDs: %s\nDecoded: %s", i, query, ids, sp.decode(ids))
    return model_file


def main(argv: Optional[Sequence[str]] = None) -> None:
    logging.basicConfig(level=logging.INFO)
    train(parser().parse_args(argv))


if __name__ == "__main__":
    main()
