"""Elastic data parallelism (scale-down): the global batch stays the same when slices are lost.

Parity targets in the reference (axlearn/common/elastic_input.py): ``ElasticSpmdInputDispatcher``
(:55-250), ``ElasticInput`` (:296-400), ``slice_count`` / ``process_count_per_slice`` (:403-420).

A job is configured for ``num_max_slices`` slices (a slice = one node's worth of feeds).  When it
runs on fewer, the feeds of the missing slices ("elastic feeds") are shared out among the
processes that are left: the missing feeds' rows are laid end to end and cut into as many
contiguous shares as there are surviving feeds, and every survivor reads its share on top of its
own feed.  Every surviving process therefore steps on ``feed_logical_batch_size +
elastic_feed_mini_batch_size`` rows and the union over processes is exactly the batch the full
job would have seen.  The runtime facts (how many slices are alive, which one this is) come from
the launcher through the config or the ``AXB_NUM_SLICES`` / ``AXB_SLICE_INDEX`` environment.
"""

from __future__ import annotations

import os
from typing import Any, Iterator, Optional

import torch

from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.input_base import Input
from axlearn_b200.common.input_dispatch import BaseInputDispatcher
from axlearn_b200.common.utils import tree_map

Tensor = torch.Tensor


def slice_count(default: int = 1) -> int:
    return int(os.environ.get("AXB_NUM_SLICES", default))


def slice_index(default: int = 0) -> int:
    return int(os.environ.get("AXB_SLICE_INDEX", default))


class ElasticSpmdInputDispatcher(BaseInputDispatcher):
    @config_class
    class Config(BaseInputDispatcher.Config):
        partition_spec: Any = None
        # The largest number of slices the job ever uses (only scaling down is supported).
        num_max_slices: Required[int] = REQUIRED
        feeds_per_slice: Required[int] = REQUIRED
        # Runtime facts; None = read from the environment.
        num_slices: Optional[int] = None
        feed_index: Optional[int] = None          # index among the feeds that are alive
        # False: feed_read_config() describes the process's own feed; True: its elastic feed.
        is_read_elastic_feed: bool = False

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        self._num_slices = cfg.num_slices if cfg.num_slices is not None else slice_count(cfg.num_max_slices)
        if self._num_slices > cfg.num_max_slices:
            raise ValueError(f"running on {self._num_slices} slices, more than num_max_slices={cfg.num_max_slices}")
        self.feed_count = cfg.feeds_per_slice * cfg.num_max_slices
        alive = cfg.feeds_per_slice * self._num_slices
        if cfg.feed_index is not None:
            self.feed_index = cfg.feed_index
        else:
            from axlearn_b200.parallel.mesh import current_mesh

            mesh = current_mesh()
            axes = mesh.present_axes(("data", "expert", "fsdp")) if mesh is not None else ()
            self.feed_index = mesh.axis_index(axes) if mesh is not None else 0
        if not 0 <= self.feed_index < alive:
            raise ValueError(f"feed_index {self.feed_index} not in [0, {alive})")
        if cfg.global_logical_batch_size % self.feed_count:
            raise ValueError(f"global_logical_batch_size {cfg.global_logical_batch_size} is not divisible by "
                             f"{self.feed_count} feeds")
        self._feed_logical_batch_size = cfg.global_logical_batch_size // self.feed_count
        # (feed, first row, end row) pieces of missing feeds that this process reads on top of
        # its own feed.
        self.elastic_segments: list[tuple[int, int, int]] = []
        self.elastic_feed_mini_batch_size = 0
        if self.is_in_elastic_mode:
            missing = self.feed_count - alive
            rows = self._feed_logical_batch_size
            # Every surviving feed takes the same number of extra rows: a contiguous range of the
            # missing feeds' rows laid end to end.
            if (missing * rows) % alive:
                raise ValueError(
                    f"{missing} missing feeds of {rows} rows cannot be shared evenly by {alive} surviving feeds")
            extra = missing * rows // alive
            self.elastic_feed_mini_batch_size = extra
            lo, hi = self.feed_index * extra, (self.feed_index + 1) * extra
            while lo < hi:
                feed, start = divmod(lo, rows)
                end = min(rows, start + hi - lo)
                self.elastic_segments.append((alive + feed, start, end))
                lo += end - start

    @property
    def elastic_feed_index(self) -> Optional[int]:
        """The (first) missing feed this process reads from, None outside elastic mode."""
        return self.elastic_segments[0][0] if self.elastic_segments else None

    @property
    def elastic_feed_mini_batch_index(self) -> int:
        if not self.elastic_segments:
            return 0
        _, start, end = self.elastic_segments[0]
        return start // max(1, end - start)

    @property
    def is_in_elastic_mode(self) -> bool:
        return self._num_slices < self._config.num_max_slices

    @property
    def num_logical_feeds(self) -> int:
        return self.feed_count

    @property
    def logical_feed_index(self) -> int:
        return self.feed_index

    @property
    def feed_logical_batch_size(self) -> int:
        return self._feed_logical_batch_size

    @property
    def partition_spec(self):
        return self._config.partition_spec

    @property
    def step_batch_size(self) -> int:
        """Rows this process steps on (its own feed plus its piece of an elastic feed)."""
        return self._feed_logical_batch_size + self.elastic_feed_mini_batch_size

    def feed_read_config(self) -> dict:
        cfg = self._config
        index = self.feed_index
        if cfg.is_read_elastic_feed and self.elastic_feed_index is not None:
            index = self.elastic_feed_index
        return dict(num_shards=self.feed_count, shard_index=index)

    def logical_to_physical_batch(self, logical_feed_batch):
        return logical_feed_batch

    def physical_to_logical_batch(self, physical_batch):
        return physical_batch

    def logical_to_physical_shapes(self, logical_feed_shapes):
        return logical_feed_shapes


class ElasticInput(Input):
    """Wraps an input config: reads the process's own feed and, in elastic mode, its piece of a
    missing slice's feed, and yields their concatenation."""

    @config_class
    class Config(Input.Config):
        input: Required[InstantiableConfig] = REQUIRED
        dispatcher: Required[InstantiableConfig] = REQUIRED
        # Name of the fields of `input` that select the shard to read.
        num_shards_field: str = "num_feeds"
        shard_index_field: str = "feed_index"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        own = cfg.dispatcher.clone(is_read_elastic_feed=False)
        self._add_child("dispatcher", own)
        self._own = self._make_input("own_input", self.dispatcher.feed_read_config())
        # One reader per missing feed this process takes rows from.
        self._elastic = [
            (self._make_input(f"elastic_input{i}", dict(num_shards=self.dispatcher.feed_count, shard_index=feed)),
             lo, hi)
            for i, (feed, lo, hi) in enumerate(self.dispatcher.elastic_segments)]

    def _make_input(self, name: str, read_cfg: dict):
        cfg = self._config
        sub = cfg.input.clone()
        setattr(sub, cfg.num_shards_field, read_cfg["num_shards"])
        setattr(sub, cfg.shard_index_field, read_cfg["shard_index"])
        return self._add_child(name, sub)

    @property
    def is_in_elastic_mode(self) -> bool:
        return self.dispatcher.is_in_elastic_mode

    def dataset(self) -> Iterator[dict]:
        if not self._elastic:
            yield from self._own.dataset()
            return
        streams = [iter(inp.dataset()) for inp, _, _ in self._elastic]
        for own in self._own.dataset():
            extras = []
            for stream, (_, lo, hi) in zip(streams, self._elastic):
                batch = next(stream, None)
                if batch is None:
                    return
                extras.append(tree_map(lambda x, lo=lo, hi=hi: x[lo:hi] if isinstance(x, Tensor) and x.dim() >= 1 else x,
                                       batch))

            def cat(a, *bs):
                if isinstance(a, Tensor) and a.dim() >= 1:
                    return torch.cat([a, *bs], dim=0)
                return a

            yield tree_map(cat, own, *extras)

    def get_state(self) -> dict:
        return {"own": self._own.get_state(), "elastic": [inp.get_state() for inp, _, _ in self._elastic]}

    def set_state(self, state: dict) -> None:
        self._own.set_state(state.get("own", {}))
        for (inp, _, _), st in zip(self._elastic, state.get("elastic", [])):
            inp.set_state(st)
