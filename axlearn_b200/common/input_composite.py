"""Inputs composed of other inputs.

Parity target: axlearn/common/input_composite.py -- ``ConcatenatedInput`` :15 (sub-inputs one after
the other; all but the last are finite) and ``ZipInput`` :44 (one batch of each sub-input per
step, under the sub-input's name; ends with the shortest).
"""

from __future__ import annotations

from typing import Iterator, Sequence

from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.input_base import Input


def _with_mode(cfg: InstantiableConfig, is_training: bool) -> InstantiableConfig:
    return cfg.clone(is_training=is_training) if "is_training" in cfg else cfg


class ConcatenatedInput(Input):
    @config_class
    class Config(Input.Config):
        is_training: Required[bool] = REQUIRED
        inputs: Sequence[InstantiableConfig] = []

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if not cfg.inputs:
            raise ValueError("Empty inputs for ConcatenatedInput")
        self._inputs = [self._add_child(f"input_{i}", _with_mode(c, cfg.is_training)) for i, c in enumerate(cfg.inputs)]

    def dataset(self) -> Iterator[dict]:
        for sub in self._inputs:
            yield from sub.dataset()


class ZipInput(Input):
    @config_class
    class Config(Input.Config):
        is_training: Required[bool] = REQUIRED
        inputs: dict = {}

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if not cfg.inputs:
            raise ValueError("Empty inputs for ZipInput")
        self._names = list(cfg.inputs)
        self._inputs = [self._add_child(f"input_{n}", _with_mode(c, cfg.is_training)) for n, c in cfg.inputs.items()]

    def dataset(self) -> Iterator[dict]:
        for parts in zip(*(sub.dataset() for sub in self._inputs)):
            yield dict(zip(self._names, parts))
