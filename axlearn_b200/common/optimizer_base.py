"""Types shared by optimizers.

Parity targets in the reference (axlearn/common/optimizer_base.py): ``OptParam`` (:30),
``OptStateSpec``, ``PartitionedGradientTransformation`` (:71).

A transformation is ``(init, update, partition)``:
``init(params) -> state``; ``update(updates, state, params) -> (updates, state)``;
``partition(param_specs) -> state specs`` (sharding of every state leaf, used by the
checkpointer and by memory accounting).  ``fused`` optionally describes the transformation in
closed form so that the learner can run it as one multi-tensor CUDA kernel over (param, grad,
mu, nu) instead of a chain of tree-wide elementwise passes; the state tree is identical either
way.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, NamedTuple, Optional, Sequence

import torch

from axlearn_b200.common.utils import TensorSpec


class OptParam(NamedTuple):
    """A parameter as seen by an optimizer."""

    value: torch.Tensor
    factorization_spec: Optional[Any] = None
    weight_decay_scale: Optional[float] = None

    @property
    def shape(self):
        return self.value.shape

    @property
    def dtype(self):
        return self.value.dtype


OptStateSpec = TensorSpec


@dataclasses.dataclass
class PartitionedGradientTransformation:
    init: Callable[[Any], Any]
    update: Callable[[Any, Any, Any], tuple[Any, Any]]
    partition: Callable[[Any], Any]
    # Closed-form description for the fused kernel path (see optimizers.FusedSpec) or None.
    fused: Optional[Any] = None

    def __iter__(self):
        # Allows ``init, update, partition = tx``.
        return iter((self.init, self.update, self.partition))


class EmptyState(NamedTuple):
    """State of stateless transformations (contributes no checkpoint leaves)."""
