"""Logical <-> physical batch dispatch.

Parity targets in the reference (axlearn/common/input_dispatch.py): ``BaseInputDispatcher`` (:28),
``InputDispatcher`` (:79-325) and ``SpmdInputDispatcher`` (:328-420).

A *feed* is a process that reads input (here: one per GPU of the batch axes).  The *logical*
global batch is what the model should see; the *physical* global batch is what the feeds can
assemble: it must divide evenly over the feeds, so when the logical batch size does not (or when
only some feeds carry data) every feed pads its share up to ``feed_physical_batch_size`` rows
and the padding is dropped again on the way into the model:

* ``feed_read_config()`` tells the local reader which shard of the source to read;
* ``logical_to_physical_batch(feed_batch)`` pads the feed's rows and attaches the bookkeeping
  (for every physical row the logical row it carries, or -1);
* ``physical_to_logical_batch(batch)`` turns an assembled physical batch back into the logical
  one.  Given a *global* physical batch it returns the global logical batch (rows ordered by
  logical feed); given one feed's physical batch it returns that feed's logical rows, which is
  what a one-process-per-GPU step consumes.

``SpmdInputDispatcher`` covers the common case in which the logical batch divides over the
ranks of the mesh's batch axes: every rank is a logical feed and the two mappings are identities.
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import TensorSpec, tree_map
from axlearn_b200.parallel.mesh import current_mesh

Tensor = torch.Tensor
PHYSICAL_TO_LOGICAL_KEY = "__physical_to_logical_batch_dispatch"


class BaseInputDispatcher(Module):
    @config_class
    class Config(Module.Config):
        global_logical_batch_size: Required[int] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True

    @property
    def num_logical_feeds(self) -> int:
        raise NotImplementedError(type(self))

    @property
    def logical_feed_index(self) -> Optional[int]:
        raise NotImplementedError(type(self))

    @property
    def feed_logical_batch_size(self) -> int:
        return self._config.global_logical_batch_size // self.num_logical_feeds

    def feed_read_config(self) -> dict:
        raise NotImplementedError(type(self))

    def logical_to_physical_batch(self, logical_feed_batch: Any) -> Any:
        raise NotImplementedError(type(self))

    def physical_to_logical_batch(self, physical_batch: Any) -> Any:
        raise NotImplementedError(type(self))

    def logical_to_physical_shapes(self, logical_feed_shapes: Any) -> Any:
        raise NotImplementedError(type(self))


def _validate_feed_batch(batch: Any, rows: int) -> None:
    from axlearn_b200.common.utils import flatten_items

    for path, x in flatten_items(batch):
        if hasattr(x, "shape") and (len(x.shape) < 1 or x.shape[0] != rows):
            raise ValueError(f"{path}: expected {rows} rows per feed, got shape {tuple(x.shape)}")


class InputDispatcher(BaseInputDispatcher):
    @config_class
    class Config(BaseInputDispatcher.Config):
        # Defaults to max(feed_logical_batch_size * num_physical_feeds, number of feeds).
        global_physical_batch_size: Optional[int] = None
        # Defaults to the number of ranks over the mesh's batch axes (1 without a mesh).
        num_physical_feeds: Optional[int] = None
        physical_feed_index: Optional[int] = None
        # logical_feed_indices[i] = the physical feed that carries logical feed i (default: as
        # many of the first feeds as divide the logical batch).
        logical_feed_indices: Optional[Sequence[int]] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        feeds, index = cfg.num_physical_feeds, cfg.physical_feed_index
        if feeds is None or index is None:
            mesh = current_mesh()
            axes = mesh.present_axes(("data", "expert", "fsdp")) if mesh is not None else ()
            feeds = feeds if feeds is not None else (mesh.axis_size(axes) if mesh is not None else 1)
            index = index if index is not None else (mesh.axis_index(axes) if mesh is not None else 0)
        self._num_physical_feeds, self._physical_feed_index = feeds, index
        if not 0 <= index < feeds:
            raise ValueError(f"physical_feed_index {index} not in [0, {feeds})")
        logical = cfg.logical_feed_indices
        if logical is None:
            n = feeds
            while cfg.global_logical_batch_size % n:
                n -= 1
            logical = list(range(n))
        logical = list(logical)
        if len(set(logical)) != len(logical) or not all(0 <= i < feeds for i in logical):
            raise ValueError(f"invalid logical_feed_indices {logical} for {feeds} physical feeds")
        if cfg.global_logical_batch_size % len(logical):
            raise ValueError(f"global_logical_batch_size {cfg.global_logical_batch_size} is not divisible by "
                             f"{len(logical)} logical feeds")
        self._logical_feed_indices = logical
        physical = cfg.global_physical_batch_size
        if physical is None:
            physical = max(self.feed_logical_batch_size * feeds, feeds)
        if physical % feeds or physical // feeds < self.feed_logical_batch_size:
            raise ValueError(f"global_physical_batch_size {physical} must be a multiple of {feeds} feeds with at "
                             f"least {self.feed_logical_batch_size} rows each")
        self._global_physical_batch_size = physical

    @property
    def num_logical_feeds(self) -> int:
        return len(self._logical_feed_indices)

    @property
    def logical_feed_index(self) -> Optional[int]:
        try:
            return self._logical_feed_indices.index(self._physical_feed_index)
        except ValueError:
            return None

    @property
    def num_physical_feeds(self) -> int:
        return self._num_physical_feeds

    @property
    def feed_physical_batch_size(self) -> int:
        return self._global_physical_batch_size // self._num_physical_feeds

    def feed_read_config(self) -> dict:
        shard = self.logical_feed_index
        if shard is None:
            # This feed's rows are dropped by physical_to_logical_batch; spread such feeds over
            # the shards anyway so that no reader is special.
            others = [i for i in range(self._num_physical_feeds) if i not in self._logical_feed_indices]
            shard = others.index(self._physical_feed_index) % self.num_logical_feeds
        return dict(num_shards=self.num_logical_feeds, shard_index=shard)

    def logical_to_physical_batch(self, logical_feed_batch: dict) -> dict:
        rows, phys = self.feed_logical_batch_size, self.feed_physical_batch_size
        _validate_feed_batch(logical_feed_batch, rows)
        feed = self.logical_feed_index

        def pad(x):
            if not isinstance(x, Tensor):
                return x
            if phys == rows:
                return x
            return torch.cat([x, x.new_zeros((phys - rows,) + tuple(x.shape[1:]))], dim=0)

        out = tree_map(pad, logical_feed_batch)
        out = dict(out)
        index = torch.full((phys,), -1, dtype=torch.int64)
        if feed is not None:
            index[:rows] = torch.arange(rows) + feed * rows
        out[PHYSICAL_TO_LOGICAL_KEY] = index
        return out

    def physical_to_logical_batch(self, physical_batch: dict) -> dict:
        batch = dict(physical_batch)
        index = batch.pop(PHYSICAL_TO_LOGICAL_KEY, None)
        if index is None:
            return batch
        keep = torch.nonzero(index >= 0).reshape(-1)
        order = keep[torch.argsort(index[keep])]

        def select(x):
            if isinstance(x, Tensor) and x.dim() >= 1 and x.shape[0] == index.shape[0]:
                return x.index_select(0, order.to(x.device))
            return x

        return tree_map(select, batch)

    def logical_to_physical_shapes(self, logical_feed_shapes: Any) -> Any:
        phys = self.feed_physical_batch_size

        def one(spec):
            return TensorSpec(shape=(phys,) + tuple(spec.shape[1:]), dtype=spec.dtype)

        out = dict(tree_map(one, logical_feed_shapes))
        out[PHYSICAL_TO_LOGICAL_KEY] = TensorSpec(shape=(phys,), dtype=torch.int64)
        return out


class SpmdInputDispatcher(BaseInputDispatcher):
    """Every rank of the batch axes is one logical feed; no padding."""

    @config_class
    class Config(BaseInputDispatcher.Config):
        partition_spec: Any = None
        num_feeds: Optional[int] = None
        feed_index: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        feeds, index = cfg.num_feeds, cfg.feed_index
        if feeds is None or index is None:
            mesh = current_mesh()
            spec = cfg.partition_spec
            axes = spec[0] if spec else ("data", "expert", "fsdp")
            axes = (axes,) if isinstance(axes, str) else tuple(axes or ())
            axes = mesh.present_axes(axes) if mesh is not None else ()
            feeds = feeds if feeds is not None else (mesh.axis_size(axes) if mesh is not None else 1)
            index = index if index is not None else (mesh.axis_index(axes) if mesh is not None else 0)
        if cfg.global_logical_batch_size % feeds:
            raise ValueError(f"partition over {feeds} feeds is incompatible with "
                             f"global_logical_batch_size={cfg.global_logical_batch_size}")
        self._feeds, self._index = feeds, index

    @property
    def num_logical_feeds(self) -> int:
        return self._feeds

    @property
    def logical_feed_index(self) -> int:
        return self._index

    @property
    def partition_spec(self):
        return self._config.partition_spec

    def feed_read_config(self) -> dict:
        return dict(num_shards=self._feeds, shard_index=self._index)

    def logical_to_physical_batch(self, logical_feed_batch):
        _validate_feed_batch(logical_feed_batch, self.feed_logical_batch_size)
        return logical_feed_batch

    def physical_to_logical_batch(self, physical_batch):
        return physical_batch

    def logical_to_physical_shapes(self, logical_feed_shapes):
        return logical_feed_shapes
