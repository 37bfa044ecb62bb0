"""Writers for inference outputs (reference: axlearn/common/inference_output.py:25-239).

An output writer receives ``(input_batch, output_batch)`` pairs whose leaves are ``[batch, ...]``
and turns every example this process holds into one record of a sink.  Two sinks: TFRecord files
of ``tf.train.Example`` protos and JSON Lines.  ``output_path`` may contain ``{data_dir}``,
``{process_index}`` and ``{process_count}``, so each process writes a file of its own.
"""

from __future__ import annotations

import json
import os
from typing import Any, Optional

import numpy as np
import torch

from axlearn_b200.common import tfrecord
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import flatten_items, get_data_dir
from axlearn_b200.parallel import collectives as coll


def _to_numpy(value: Any) -> Any:
    if isinstance(value, torch.Tensor):
        value = value.detach()
        if value.dtype in (torch.bfloat16, torch.float16):
            value = value.float()
        return value.cpu().numpy()
    return value


def _index_tree(tree: Any, i: int) -> Any:
    if isinstance(tree, dict):
        return {k: _index_tree(v, i) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)) and not (tree and isinstance(tree[0], (str, bytes))):
        return type(tree)(_index_tree(v, i) for v in tree)
    return tree[i]


def _batch_size(tree: Any) -> Optional[int]:
    if isinstance(tree, dict):
        for v in tree.values():
            n = _batch_size(v)
            if n is not None:
                return n
        return None
    if isinstance(tree, (torch.Tensor, np.ndarray)):
        return tree.shape[0] if tree.ndim else None
    if isinstance(tree, (list, tuple)):
        return len(tree)
    return None


def _format_path(template: str) -> str:
    try:
        data_dir = get_data_dir()
    except Exception:  # pylint: disable=broad-except
        data_dir = ""
    return template.format(data_dir=data_dir, process_index=coll.process_index(), process_count=coll.process_count())


class BaseOutputWriter(Module):
    """Writes records for inference outputs."""

    @config_class
    class Config(Module.Config):
        # How the batch dimension is spread over processes.  Every process of this runtime holds
        # its own slice of the batch, which is what the reference calls FULL; kept so that configs
        # carry over.
        batch_partition_spec: Any = "FULL"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    def write(self, *, input_batch: dict, output_batch: Any) -> None:
        raise NotImplementedError(type(self))

    def flush(self) -> None:
        raise NotImplementedError(type(self))


class BaseRecordSink(Module):
    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    def write(self, record: Any) -> None:
        raise NotImplementedError(type(self))

    def flush(self) -> None:
        raise NotImplementedError(type(self))


def _tf_feature(value: Any) -> Any:
    value = _to_numpy(value)
    if isinstance(value, (bytes, str)):
        return [value]
    arr = np.asarray(value)
    if arr.dtype.kind in "fbiuSUO":
        return arr.reshape(-1)
    raise NotImplementedError(f"{arr.dtype}: {value}")


def _json_feature(value: Any) -> Any:
    value = _to_numpy(value)
    if isinstance(value, bytes):
        return value.decode("utf-8")
    if isinstance(value, np.ndarray):
        if value.dtype.kind in "SO":
            value = np.char.decode(value.astype(np.bytes_), "utf-8")
        return value.tolist()
    if isinstance(value, np.generic):
        return value.item()
    return value


class TfExampleRecordSink(BaseRecordSink):
    """Each record becomes one ``tf.train.Example`` in a TFRecord file; the feature names are the
    ``/``-joined paths of the record's leaves."""

    @config_class
    class Config(BaseRecordSink.Config):
        output_path: Required[str] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self.output_path = _format_path(cfg.output_path)
        os.makedirs(os.path.dirname(self.output_path) or ".", exist_ok=True)
        self._writer = tfrecord.TFRecordWriter(self.output_path)

    def write(self, record: Any) -> None:
        self._writer.write(tfrecord.encode_example({path: _tf_feature(v) for path, v in flatten_items(record)}))

    def flush(self) -> None:
        self._writer.flush()


class JsonlExampleRecordSink(BaseRecordSink):
    """Each record becomes one line ``{path: value}`` of a JSON Lines file."""

    @config_class
    class Config(BaseRecordSink.Config):
        output_path: Required[str] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self.output_path = _format_path(cfg.output_path)
        os.makedirs(os.path.dirname(self.output_path) or ".", exist_ok=True)
        self._writer = open(self.output_path, "w", encoding="utf-8")  # pylint: disable=consider-using-with

    def write(self, record: Any) -> None:
        self._writer.write(json.dumps({path: _json_feature(v) for path, v in flatten_items(record)}) + "\n")

    def flush(self) -> None:
        self._writer.flush()


class OutputRecordWriter(BaseOutputWriter):
    """Writes each example's OUTPUT as a record of ``sink``.  The examples a process holds are
    disjoint from every other process's, so no coordination is needed."""

    @config_class
    class Config(BaseOutputWriter.Config):
        sink: BaseRecordSink.Config = TfExampleRecordSink.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("sink", cfg.sink)

    def write(self, *, input_batch: dict, output_batch: Any) -> None:
        data = dict(input=input_batch, output=output_batch)
        n = _batch_size(data)
        if n is None:
            raise ValueError("no leaf with a batch dimension")
        for i in range(n):
            example = _index_tree(data, i)
            self.sink.write(self._build_record(input_example=example["input"], output_example=example["output"]))

    def _build_record(self, *, input_example: Any, output_example: Any) -> Any:
        del input_example
        return output_example

    def flush(self) -> None:
        self.sink.flush()


class InputOutputRecordWriter(OutputRecordWriter):
    """Writes both sides of each example, under ``input`` and ``output``."""

    def _build_record(self, *, input_example: Any, output_example: Any) -> Any:
        return dict(input=input_example, output=output_example)
