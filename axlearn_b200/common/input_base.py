"""Input pipeline contract.

Parity targets in the reference (axlearn/common/input_base.py): ``partition_by_path_rank``
(:50-119), ``Input`` (:122) with ``dataset()`` (:196), ``batches()`` (:213),
``dispatch_global_batch()`` (:227), ``element_spec()`` (:277), ``partition_spec``.

Each process feeds only its own GPU.  ``batches()`` yields *per-process* batches (global batch
divided by the number of data-parallel feeds); tensors are produced in pinned host memory so
that the trainer's host→device copy is asynchronous.
"""

from __future__ import annotations

import re
from typing import Any, Iterable, Iterator, Optional, Sequence

import torch

from axlearn_b200.common.config import InstantiableConfig, config_class
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import PartitionSpec, flatten_items, tree_map


class PathAndRank:
    """Rule: tensors whose path matches ``path_regex`` and rank equals ``rank`` (None = any)."""

    def __init__(self, path_regex: str, rank: Optional[int]):
        self.path_regex, self.rank = path_regex, rank


def partition_by_path_rank(path_rank_to_partition: Sequence[tuple[PathAndRank, Any]]):
    """Returns ``tree -> tree of PartitionSpec`` by the first matching (path, rank) rule."""

    def fn(tree: Any) -> Any:
        def pick(path: str, x: Any):
            rank = len(x.shape)
            for rule, spec in path_rank_to_partition:
                if re.fullmatch(rule.path_regex, path) and (rule.rank is None or rule.rank == rank):
                    return spec
            return None

        items = flatten_items(tree)
        from axlearn_b200.common.utils import unflatten_items

        return unflatten_items([(p, pick(p, v)) for p, v in items])

    return fn


class Input(Module):
    """Produces batches for training or evaluation."""

    @config_class
    class Config(Module.Config):
        # Mesh axes of the batch dim of every input tensor.
        partition_spec: Optional[Any] = None
        input_dispatcher: Optional[InstantiableConfig] = None
        input_partitioner: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        if cfg.input_dispatcher is not None:
            self._add_child("input_dispatcher", cfg.input_dispatcher)

    def dataset(self) -> Iterable[dict]:
        """An iterable of per-process batches."""
        raise NotImplementedError(type(self))

    def __iter__(self) -> Iterator[dict]:
        return iter(self.dataset())

    def batches(self, it: Iterator[dict]) -> Iterator[dict]:
        """Yields batches from ``it``, mapping logical to physical batches when a dispatcher
        is configured."""
        for batch in it:
            if "input_dispatcher" in self._children:
                batch = self.input_dispatcher.logical_to_physical_batch(batch)
            yield batch

    def dispatch_global_batch(self, global_physical_batch: dict, *, batch_axis_names: Any = "data") -> dict:
        """Device-side half of dispatch: physical → logical batch (drops padding rows)."""
        if "input_dispatcher" in self._children:
            return self.input_dispatcher.physical_to_logical_batch(global_physical_batch)
        return global_physical_batch

    def element_spec(self) -> dict:
        """Shapes/dtypes of one per-process batch."""
        batch = next(iter(self.dataset()))
        from axlearn_b200.common.utils import TensorSpec

        return tree_map(lambda x: TensorSpec(shape=tuple(x.shape), dtype=x.dtype), batch)

    # Checkpointable iterator state (overridden by stateful inputs).
    def get_state(self) -> dict:
        return {}

    def set_state(self, state: dict) -> None:
        del state
