"""Synthetic inputs.

Parity targets in the reference (axlearn/common/input_fake.py): ``EmptyInput`` (:22),
``FakeLmInput`` (:60-88) — ``tokens = randint([B_local, T+1], 0, max_token_id)``,
``input_ids = tokens[:, :-1]``, ``target_labels = tokens[:, 1:]``,
``target_num_bytes = ones`` — and ``FakeSeq2SeqInput`` (:91).

Batches are generated on the host into pinned memory from a counter-based key
(seed, process index, batch index), so a resumed run regenerates exactly the same stream
from its saved batch index.
"""

from __future__ import annotations

from typing import Iterator, Optional, Sequence

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.input_base import Input
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import current_mesh


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except RuntimeError:
            return t
    return t


class EmptyInput(Input):
    """Yields empty batches forever (for models that generate their own data)."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        total_num_batches: Optional[int] = None

    def dataset(self):
        n = self._config.total_num_batches
        i = 0
        while n is None or i < n:
            yield {}
            i += 1


class FakeLmInput(Input):
    """Uniform-random token LM batches."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        global_batch_size: Required[int] = REQUIRED
        source_length: Required[int] = REQUIRED
        vocab_size: int = 32768
        seed: int = 0
        total_num_batches: Optional[int] = None
        # Number of data-parallel feeds; None = from the mesh in scope (product of batch axes).
        num_feeds: Optional[int] = None
        feed_index: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._batch_index = 0
        # The mesh in scope at construction (the trainer builds its children inside its mesh)
        # decides which rows of the global batch this process feeds; iterating the dataset
        # later, outside any mesh context, must not change that.
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

    def dataset(self) -> Iterator[dict]:
        cfg = self._config
        feeds, index = self._feeds()
        if cfg.global_batch_size % feeds:
            raise ValueError(f"global batch {cfg.global_batch_size} not divisible by {feeds} feeds")
        local = cfg.global_batch_size // feeds
        base = prng.PRNGKey(cfg.seed)
        if not cfg.is_training:
            # An evaluation input is iterated from the start every time (each evaluation sees the
            # same batches); a training input continues where its state says.
            self._batch_index = 0
        while cfg.total_num_batches is None or self._batch_index < cfg.total_num_batches:
            # The global batch is a function of (seed, batch index) only; each feed takes its
            # rows, so the data does not depend on how many ranks share the batch.
            key = prng.fold_in(base, self._batch_index)
            tokens = prng.randint(
                key, (cfg.global_batch_size, cfg.source_length + 1), 0, cfg.vocab_size, dtype=torch.int32)
            tokens = tokens[index * local:(index + 1) * local]
            self._batch_index += 1
            yield {
                "input_ids": _pin(tokens[:, :-1].contiguous()),
                "target_labels": _pin(tokens[:, 1:].contiguous()),
                "target_num_bytes": _pin(torch.ones(local, dtype=torch.int32)),
            }

    def get_state(self) -> dict:
        return {"batch_index": self._batch_index}

    def set_state(self, state: dict) -> None:
        self._batch_index = int(state.get("batch_index", 0))


class FakeSeq2SeqInput(Input):
    """Random source/target id pairs for encoder-decoder models."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        global_batch_size: Required[int] = REQUIRED
        source_length: Required[int] = REQUIRED
        target_length: Required[int] = REQUIRED
        vocab_size: int = 32768
        seed: int = 0
        total_num_batches: Optional[int] = None

    def dataset(self):
        cfg = self._config
        i = 0
        base = prng.fold_in(prng.PRNGKey(cfg.seed), coll.process_index())
        local = cfg.global_batch_size // max(1, coll.process_count())
        while cfg.total_num_batches is None or i < cfg.total_num_batches:
            k1, k2 = prng.split(prng.fold_in(base, i), 2)
            src = prng.randint(k1, (local, cfg.source_length), 1, cfg.vocab_size)
            tgt = prng.randint(k2, (local, cfg.target_length + 1), 1, cfg.vocab_size)
            i += 1
            yield {
                "source": {"input_ids": src},
                "target": {"input_ids": tgt[:, :-1].contiguous()},
                "target_labels": tgt[:, 1:].contiguous(),
            }


class FakeImageInput(Input):
    """Random ``{"image": [B, H, W, 3], "label": [B]}`` batches (reference:
    axlearn/vision/input_image.py ``fake_image_dataset``)."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        global_batch_size: Required[int] = REQUIRED
        image_size: Sequence[int] = (224, 224)
        num_classes: int = 1000
        seed: int = 0
        total_num_batches: Optional[int] = None

    def dataset(self):
        cfg = self._config
        base = prng.fold_in(prng.PRNGKey(cfg.seed), coll.process_index())
        local = cfg.global_batch_size // max(1, coll.process_count())
        i = 0
        while cfg.total_num_batches is None or i < cfg.total_num_batches:
            k1, k2 = prng.split(prng.fold_in(base, i), 2)
            image = prng.normal(k1, (local, *cfg.image_size, 3))
            label = prng.randint(k2, (local,), 0, cfg.num_classes)
            i += 1
            yield {"image": _pin(image), "label": _pin(label)}


class FakeSpeechInput(Input):
    """Random waveforms of random lengths with label sequences: ``inputs [B, samples]``,
    ``paddings``, ``target_labels`` (labels, EOS, then -1) and ``target.input_ids`` (BOS, labels)."""

    @config_class
    class Config(Input.Config):
        is_training: bool = True
        global_batch_size: Required[int] = REQUIRED
        max_source_len: int = 16000
        max_target_len: int = 16
        vocab_size: int = 1024
        bos_id: int = 1
        eos_id: int = 2
        seed: int = 0
        total_num_batches: Optional[int] = None

    def dataset(self):
        cfg = self._config
        base = prng.fold_in(prng.PRNGKey(cfg.seed), coll.process_index())
        local = cfg.global_batch_size // max(1, coll.process_count())
        i = 0
        while cfg.total_num_batches is None or i < cfg.total_num_batches:
            k1, k2, k3, k4 = prng.split(prng.fold_in(base, i), 4)
            wave = prng.normal(k1, (local, cfg.max_source_len))
            n = prng.randint(k2, (local,), cfg.max_source_len // 2, cfg.max_source_len + 1)
            paddings = torch.arange(cfg.max_source_len)[None] >= n[:, None]
            u = prng.randint(k3, (local,), 1, cfg.max_target_len)
            tokens = prng.randint(k4, (local, cfg.max_target_len), 3, cfg.vocab_size)
            pos = torch.arange(cfg.max_target_len)[None]
            labels = torch.where(pos < u[:, None], tokens, torch.full_like(tokens, -1))
            labels = torch.where(pos == u[:, None], torch.full_like(tokens, cfg.eos_id), labels)
            ids = torch.cat([torch.full((local, 1), cfg.bos_id, dtype=tokens.dtype), tokens[:, :-1]], dim=1)
            ids = torch.where(pos <= u[:, None], ids, torch.zeros_like(ids))
            i += 1
            yield {"inputs": _pin(wave * (~paddings)), "paddings": _pin(paddings),
                   "target_labels": _pin(labels), "target": {"input_ids": _pin(ids)}}
