"""Update transformations: wrappers that decide *whether* and *how* an optimizer's updates apply.

Parity targets in the reference (axlearn/common/update_transformation.py):
``WrappedPartitionedGradientTransformation`` (:75), ``ConditionalUpdateTransformation`` (:122:
run the inner transformation only every ``update_every_k`` steps; in between nothing changes) and
``OverrideInplaceUpdateTransformation`` (:380: for parameters whose path matches a rule, the
"gradient" *is* the new value -- used by delayed-scaling fp8, whose scale / amax-history
parameters return their next value through the backward pass).

Here they are ordinary ``PartitionedGradientTransformation`` wrappers, so they compose with
``chain`` and plug into ``Learner.Config.optimizer`` like any optimizer.  The config classes with
the reference's names instantiate to those wrappers.
"""

from __future__ import annotations

import re
from typing import Any, NamedTuple, Optional, Sequence

import torch

from axlearn_b200.common.config import REQUIRED, Configurable, InstantiableConfig, Required, config_class, maybe_instantiate
from axlearn_b200.common.optimizer_base import OptParam, PartitionedGradientTransformation
from axlearn_b200.common.utils import TensorSpec, flatten_items, tree_map, tree_paths, unflatten_items

Tensor = torch.Tensor


def _is_leaf(x: Any) -> bool:
    return x is None or isinstance(x, (Tensor, OptParam, TensorSpec))


class ConditionalState(NamedTuple):
    count: Tensor
    inner: Any


def conditional_update(inner: Any, *, update_every_k: int = 1, start_step: int = 0) -> PartitionedGradientTransformation:
    """Runs ``inner`` at the 1-based steps ``t >= start_step`` with ``t % update_every_k == 0``;
    at other steps the updates are zero and the inner state is left untouched."""
    inner = maybe_instantiate(inner)

    def init(params):
        return ConditionalState(torch.zeros((), dtype=torch.int32), inner.init(params))

    def update(updates, state, params=None):
        count = state.count + 1
        t = int(count)
        if t >= start_step and t % update_every_k == 0:
            out, inner_state = inner.update(updates, state.inner, params)
            return out, ConditionalState(count, inner_state)
        zeros = tree_map(lambda u: None if u is None else torch.zeros_like(u), updates, is_leaf=_is_leaf)
        return zeros, ConditionalState(count, state.inner)

    def partition(specs):
        return ConditionalState(TensorSpec(shape=(), dtype=torch.int32), inner.partition(specs))

    return PartitionedGradientTransformation(init, update, partition)


def override_inplace_update(inner: Any, *, rules: Sequence[str]) -> PartitionedGradientTransformation:
    """Parameters whose path fully matches one of ``rules`` take their incoming "gradient" as
    their new value (update = value - parameter), bypassing ``inner``; all other parameters go
    through ``inner`` (which sees ``None`` for the overridden ones)."""
    inner = maybe_instantiate(inner)
    patterns = [re.compile(r) for r in rules]

    def overridden(path: str) -> bool:
        return any(p.fullmatch(path) for p in patterns)

    def split(tree):
        paths = tree_paths(tree, is_leaf=_is_leaf)
        return tree_map(lambda x, p: None if overridden(p) else x, tree, paths, is_leaf=_is_leaf)

    def update(updates, state, params=None):
        if params is None:
            raise ValueError("override_inplace_update requires params")
        rest, new_state = inner.update(split(updates), state, params)
        flat_rest = dict(flatten_items(rest, is_leaf=_is_leaf))
        flat_params = dict(flatten_items(params, is_leaf=_is_leaf))
        out = []
        for path, g in flatten_items(updates, is_leaf=_is_leaf):
            if g is not None and overridden(path):
                p = flat_params[path]
                value = p.value if isinstance(p, OptParam) else p
                out.append((path, g.to(value.dtype) - value))
            else:
                out.append((path, flat_rest.get(path)))
        return unflatten_items(out), new_state

    # No optimizer state exists for the overridden parameters (reference:
    # axlearn/common/update_transformation.py:415-424).
    def init(params):
        return inner.init(split(params))

    def partition(specs):
        return inner.partition(split(specs))

    return PartitionedGradientTransformation(init, update, partition)


class UpdateTransformation(Configurable):
    """Base of the config classes below: ``cfg.instantiate()`` yields the transformation."""

    @config_class
    class Config(Configurable.Config):
        pass


class WrappedPartitionedGradientTransformation(UpdateTransformation):
    @config_class
    class Config(UpdateTransformation.Config):
        transformation: Required[Any] = REQUIRED

    def __new__(cls, cfg):
        return maybe_instantiate(cfg.transformation)


class ConditionalUpdateTransformation(UpdateTransformation):
    @config_class
    class Config(UpdateTransformation.Config):
        inner: Required[Any] = REQUIRED
        update_every_k: int = 1
        start_step: int = 0

    def __new__(cls, cfg):
        return conditional_update(cfg.inner, update_every_k=cfg.update_every_k, start_step=cfg.start_step)


class OverrideInplaceUpdateTransformation(UpdateTransformation):
    @config_class
    class Config(UpdateTransformation.Config):
        transformation: Required[Any] = REQUIRED
        rules: Sequence[str] = []

    def __new__(cls, cfg):
        return override_inplace_update(cfg.transformation, rules=cfg.rules)
