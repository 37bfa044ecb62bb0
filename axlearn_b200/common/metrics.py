"""Summaries that know how to be averaged across steps and ranks.

Parity targets in the reference (axlearn/common/metrics.py): ``WeightedSummary`` (:35) and
its Min/Max/Sum relatives, ``MetricAccumulator`` (:122).
"""

from __future__ import annotations

import dataclasses
from typing import Any, Optional, Union

import torch

Scalar = Union[float, int, torch.Tensor]


def _f(x: Scalar) -> float:
    if isinstance(x, torch.Tensor):
        return float(x.detach().float().item()) if x.numel() == 1 else x.detach().float()
    return float(x)


@dataclasses.dataclass
class MetricSummary:
    def value(self) -> Any:
        raise NotImplementedError

    def accumulate(self, other: "MetricSummary") -> "MetricSummary":
        raise NotImplementedError


@dataclasses.dataclass
class WeightedSummary(MetricSummary):
    """A mean with the weight (count) it was taken over; accumulation is a weighted mean."""

    mean: Scalar
    weight: Scalar

    def value(self):
        return self.mean

    def accumulate(self, other: "WeightedSummary") -> "WeightedSummary":
        w0, w1 = _f(self.weight), _f(other.weight)
        total = w0 + w1
        if total == 0:
            return WeightedSummary(0.0, 0.0)
        return WeightedSummary((_f(self.mean) * w0 + _f(other.mean) * w1) / total, total)


# The reference's historical name.
WeightedScalar = WeightedSummary


@dataclasses.dataclass
class MinSummary(MetricSummary):
    _value: Scalar

    def value(self):
        return self._value

    def accumulate(self, other):
        return MinSummary(min(_f(self._value), _f(other._value)))


@dataclasses.dataclass
class MaxSummary(MetricSummary):
    _value: Scalar

    def value(self):
        return self._value

    def accumulate(self, other):
        return MaxSummary(max(_f(self._value), _f(other._value)))


@dataclasses.dataclass
class SumSummary(MetricSummary):
    _value: Scalar

    def value(self):
        return self._value

    def accumulate(self, other):
        return SumSummary(_f(self._value) + _f(other._value))


class MetricAccumulator:
    """Accumulates trees of summaries across calls to ``update``."""

    def __init__(self):
        self._acc: Optional[dict] = None

    @classmethod
    def default_config(cls):
        from axlearn_b200.common.config import config_for_class

        return config_for_class(cls)

    def update(self, summaries: dict) -> None:
        from axlearn_b200.common.utils import flatten_items

        flat = dict(flatten_items(summaries, is_leaf=lambda x: isinstance(x, MetricSummary)))
        flat = {k: v for k, v in flat.items() if isinstance(v, MetricSummary)}
        if self._acc is None:
            self._acc = flat
            return
        for k, v in flat.items():
            self._acc[k] = self._acc[k].accumulate(v) if k in self._acc else v

    def summaries(self) -> dict:
        from axlearn_b200.common.utils import unflatten_items

        return unflatten_items(list((self._acc or {}).items()))
