"""Text -> language-model training / evaluation / decoding inputs.

Parity targets in the reference: ``text_to_lm_training_input`` (axlearn/common/input_lm.py:56-232:
tokenize, concatenate documents separated by EOS, cut the stream into ``max_len`` chunks, either
plain -- ``EOS_DELIM_NO_MASK`` -- or with per-document segment ids and positions --
``EOS_DELIM_MASK``; drop or pad the tail by ``max_padding_fraction``; shuffle),
``text_to_lm_eval_input`` (:235-383: strided windows with only the new tokens counted as
targets), ``lm_decoding_prefix_processor`` (:1083), ``PackingMethodType`` (:42) and the
sentencepiece vocabularies under ``axlearn/data/tokenizers``.

The reference builds these as tf.data / seqio graphs; here they are plain Python generators over
any iterable of ``{"text": str}`` examples, batched by ``TextLmInput`` into pinned per-process
tensors.  Document order, packing and the (seeded) shuffle are deterministic and the reader
position is checkpointable, so a resumed run continues with the next unseen batch.
"""

from __future__ import annotations

import enum
import random
from typing import Any, Callable, Iterable, Iterator, Optional, Sequence

import torch

from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class
from axlearn_b200.common.input_base import Input
from axlearn_b200.parallel.mesh import current_mesh


class PackingMethodType(enum.Enum):
    # Documents are concatenated with EOS in between; attention may cross documents.
    EOS_DELIM_NO_MASK = "eos_delim_no_mask"
    # As above, plus segment ids / positions so that attention and RoPE restart per document.
    EOS_DELIM_MASK = "eos_delim_mask"


# ------------------------------------------------------------------------------------------
# Vocabularies.
# ------------------------------------------------------------------------------------------


class SentencePieceVocabulary(Configurable):
    """A sentencepiece model file (the reference's ``seqio.SentencePieceVocabulary``)."""

    @config_class
    class Config(Configurable.Config):
        sentencepiece_model_file: Required[str] = REQUIRED
        eos_id: Optional[int] = None
        pad_id: int = 0

    def __init__(self, cfg):
        super().__init__(cfg)
        import sentencepiece as spm  # pylint: disable=import-outside-toplevel

        self._sp = spm.SentencePieceProcessor(model_file=cfg.sentencepiece_model_file)

    @property
    def vocab_size(self) -> int:
        return self._sp.get_piece_size()

    @property
    def eos_id(self) -> int:
        return self._config.eos_id if self._config.eos_id is not None else self._sp.eos_id()

    @property
    def pad_id(self) -> int:
        return self._config.pad_id

    def encode(self, text: str) -> list[int]:
        return list(self._sp.encode(text))

    def decode(self, ids: Sequence[int]) -> str:
        return self._sp.decode([int(i) for i in ids])


class ByteVocabulary(Configurable):
    """UTF-8 bytes shifted by ``offset`` (ids below it are pad / EOS / unused): needs no model
    file, handy for tests and byte-level models."""

    @config_class
    class Config(Configurable.Config):
        offset: int = 3
        eos_id: int = 1
        pad_id: int = 0

    @property
    def vocab_size(self) -> int:
        return 256 + self._config.offset

    @property
    def eos_id(self) -> int:
        return self._config.eos_id

    @property
    def pad_id(self) -> int:
        return self._config.pad_id

    def encode(self, text: str) -> list[int]:
        return [b + self._config.offset for b in text.encode("utf-8")]

    def decode(self, ids: Sequence[int]) -> str:
        off = self._config.offset
        return bytes(int(i) - off for i in ids if int(i) >= off).decode("utf-8", errors="replace")


# ------------------------------------------------------------------------------------------
# Example-level processors (generators of dicts of int lists).
# ------------------------------------------------------------------------------------------


def text_to_lm_training_input(
    examples: Iterable[dict],
    *,
    vocab: Any,
    max_len: int,
    replace_newlines_with: str = "\n",
    window_size: int = 128,
    max_padding_fraction: float = 1.0,
    shuffle_buffer_size: int = 0,
    packing_method: Optional[PackingMethodType] = None,
    seed: int = 0,
) -> Iterator[dict]:
    """Yields ``{"input_ids", "target_labels", "target_num_bytes"[, "input_segment_ids",
    "input_positions"]}`` of length ``max_len`` from ``{"text": ...}`` examples.

    ``window_size`` documents are tokenised and concatenated (EOS first, between documents and
    last); the stream is cut into ``max_len`` chunks; a final partial chunk is padded if that
    needs at most ``max_padding_fraction * max_len`` padding, else dropped.  Targets are the
    inputs shifted by one inside the chunk's stream (the token after the last input of a chunk is
    the first token of the next chunk, or padding).
    """
    assert 0.0 <= max_padding_fraction <= 1.0
    method = packing_method or PackingMethodType.EOS_DELIM_NO_MASK
    eos, pad = vocab.eos_id, vocab.pad_id
    rng = random.Random(seed)
    buffer: list[dict] = []

    def emit(ex):
        if shuffle_buffer_size <= 1:
            yield ex
            return
        buffer.append(ex)
        if len(buffer) >= shuffle_buffer_size:
            yield buffer.pop(rng.randrange(len(buffer)))

    def chunks_of(window: list[str]):
        stream, segments = [eos], [0]
        for d, text in enumerate(window):
            ids = vocab.encode(text.replace("\n", replace_newlines_with))
            stream.extend(ids + [eos])
            segments.extend([d + 1] * (len(ids) + 1))
        n_full, rest = divmod(len(stream) - 1, max_len)
        total = n_full
        if rest and (max_len - rest) <= max_padding_fraction * max_len:
            total += 1
        for c in range(total):
            lo = c * max_len
            inp = stream[lo:lo + max_len]
            tgt = stream[lo + 1:lo + 1 + max_len]
            seg = segments[lo:lo + max_len]
            valid = len(tgt)
            inp = inp + [pad] * (max_len - len(inp))
            tgt = tgt + [pad] * (max_len - len(tgt))
            ex = {
                "input_ids": inp, "target_labels": tgt,
                "target_num_bytes": len(vocab.decode([t for t in tgt[:valid] if t not in (eos, pad)]).encode("utf-8")),
            }
            if method == PackingMethodType.EOS_DELIM_MASK:
                # Segment ids count documents from 1 within the chunk (0 = padding); positions
                # restart at every document boundary.
                n_in = len(stream[lo:lo + max_len])
                seg_ids, positions, remap, last = [], [], {}, None
                for i in range(max_len):
                    if i >= n_in:
                        seg_ids.append(0)
                        positions.append(0)
                        continue
                    doc = seg[i]
                    remap.setdefault(doc, len(remap) + 1)
                    seg_ids.append(remap[doc])
                    positions.append(positions[-1] + 1 if doc == last else 0)
                    last = doc
                ex["input_segment_ids"] = seg_ids
                ex["input_positions"] = positions
            yield ex

    window: list[str] = []
    for example in examples:
        window.append(example["text"])
        if len(window) == window_size:
            for ch in chunks_of(window):
                yield from emit(ch)
            window = []
    if window:
        for ch in chunks_of(window):
            yield from emit(ch)
    while buffer:
        yield buffer.pop(rng.randrange(len(buffer)))


def text_to_lm_eval_input(
    examples: Iterable[dict],
    *,
    vocab: Any,
    max_len: int,
    replace_newlines_with: str = "\n",
    stride: Optional[int] = None,
) -> Iterator[dict]:
    """Strided evaluation windows over each document: every window has ``max_len`` inputs, but
    only the tokens not scored by an earlier window are live targets (the others are set to the
    padding id), so each token is scored once with up to ``max_len - stride`` tokens of context."""
    eos, pad = vocab.eos_id, vocab.pad_id
    stride = stride or max_len
    assert 0 < stride <= max_len
    for example in examples:
        ids = [eos] + vocab.encode(example["text"].replace("\n", replace_newlines_with)) + [eos]
        n = len(ids) - 1
        scored = 0
        start = 0
        while scored < n:
            end = min(start + max_len, n)
            inp = ids[start:end]
            tgt = ids[start + 1:end + 1]
            tgt = [pad if start + i < scored else t for i, t in enumerate(tgt)]
            live = [t for t in tgt if t not in (pad, eos)]
            scored = end
            yield {
                "input_ids": inp + [pad] * (max_len - len(inp)),
                "target_labels": tgt + [pad] * (max_len - len(tgt)),
                "target_num_bytes": len(vocab.decode(live).encode("utf-8")),
            }
            if end == n:
                break
            start += stride


def lm_decoding_prefix_processor(examples: Iterable[dict], *, vocab: Any, max_len: int) -> Iterator[dict]:
    """``{"text"}`` -> ``{"prefix"}``: EOS (as the conditioning token) + the tokenised prompt,
    left-truncated to ``max_len`` and right-padded."""
    for example in examples:
        ids = ([vocab.eos_id] + vocab.encode(example["text"]))[-max_len:]
        yield {"prefix": ids + [vocab.pad_id] * (max_len - len(ids))}


# ------------------------------------------------------------------------------------------
# Batching input.
# ------------------------------------------------------------------------------------------


class TextLmInput(Input):
    """Batches a processed example stream into per-process tensors.

    ``source`` is a config (or zero-argument callable) producing the raw example iterable;
    ``processor`` maps it to fixed-length examples (e.g. ``text_to_lm_training_input`` with its
    arguments bound through ``config_for_function``-style partial application).  Global batch
    ``b`` consists of processed examples ``[b * B, (b + 1) * B)``; every feed keeps its rows."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        global_batch_size: Required[int] = REQUIRED
        source: Required[Any] = REQUIRED
        processor: Required[Any] = REQUIRED
        repeat: bool = True
        total_num_batches: Optional[int] = None
        num_feeds: Optional[int] = None
        feed_index: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._batch_index = 0
        self._mesh = current_mesh()

    def _feeds(self) -> tuple[int, int]:
        cfg = self._config
        if cfg.num_feeds is not None:
            return cfg.num_feeds, cfg.feed_index or 0
        mesh = self._mesh or current_mesh()
        if mesh is None:
            return 1, 0
        axes = mesh.present_axes(("data", "expert", "fsdp"))
        return mesh.axis_size(axes), mesh.axis_index(axes)

    def _examples(self) -> Iterator[dict]:
        cfg = self._config
        while True:
            src = cfg.source.instantiate() if isinstance(cfg.source, InstantiableConfig) else cfg.source()
            proc = cfg.processor.instantiate() if isinstance(cfg.processor, InstantiableConfig) else cfg.processor
            produced = False
            for ex in proc(src):
                produced = True
                yield ex
            if not cfg.repeat or not produced:
                return

    def dataset(self) -> Iterator[dict]:
        cfg = self._config
        feeds, index = self._feeds()
        if cfg.global_batch_size % feeds:
            raise ValueError(f"global batch {cfg.global_batch_size} not divisible by {feeds} feeds")
        local = cfg.global_batch_size // feeds
        it = self._examples()
        # Resume: skip what earlier batches consumed.
        for _ in range(self._batch_index * cfg.global_batch_size):
            if next(it, None) is None:
                return
        while cfg.total_num_batches is None or self._batch_index < cfg.total_num_batches:
            rows = []
            for _ in range(cfg.global_batch_size):
                ex = next(it, None)
                if ex is None:
                    return
                rows.append(ex)
            self._batch_index += 1
            mine = rows[index * local:(index + 1) * local]
            batch = {}
            for key in mine[0]:
                t = torch.tensor([r[key] for r in mine], dtype=torch.int32)
                batch[key] = t.pin_memory() if torch.cuda.is_available() else t
            yield batch

    def get_state(self) -> dict:
        return {"batch_index": self._batch_index}

    def set_state(self, state: dict) -> None:
        self._batch_index = int(state.get("batch_index", 0))
