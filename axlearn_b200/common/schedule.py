"""Learning-rate / scale schedules: ``step -> float``.

Schedules are plain host-side functions of the (1-based, when driven by the optimizers) step;
their value is passed to the fused optimizer kernel as a scalar argument.

Parity targets in the reference (axlearn/common/schedule.py): ``polynomial`` (:36),
``exponential`` (:75), ``inverse_sqrt`` (:117), ``adafactor`` (:135), ``stepwise`` (:211),
``segment_wise`` (:254), ``cosine_with_linear_warmup`` (:301), ``warmup_stable_decay``
(:357), ``constant_with_linear_warmup`` (:412), ``linear_schedule_with_warmup`` (:444),
``ema_schedule`` (:481).
"""

from __future__ import annotations

import math
from typing import Callable, Optional, Sequence, Union

from axlearn_b200.common.config import InstantiableConfig, maybe_instantiate

ScheduleFn = Callable[[Union[int, float]], float]
Schedule = Union[float, int, ScheduleFn, InstantiableConfig]


def as_schedule_fn(s: Optional[Schedule]) -> ScheduleFn:
    """Constants become constant schedules; configs are instantiated."""
    s = maybe_instantiate(s)
    if s is None:
        return lambda step: 1.0
    if callable(s):
        return s
    value = float(s)
    return lambda step: value


def constant_schedule(value: float) -> ScheduleFn:
    return lambda step: float(value)


def polynomial(*, begin_step: int = 0, begin_value: float = 0.0, end_step: int, end_value: float,
               power: float = 1.0) -> ScheduleFn:
    """``begin_value`` before ``begin_step``, ``end_value`` after ``end_step``, and
    ``begin + (end - begin) * frac**power`` in between."""

    def fn(step):
        if end_step <= begin_step:
            return float(end_value if step >= end_step else begin_value)
        frac = min(1.0, max(0.0, (step - begin_step) / (end_step - begin_step)))
        return float(begin_value + (end_value - begin_value) * frac**power)

    return fn


def exponential(*, begin_step: int = 0, begin_value: float, end_step: int, end_value: float) -> ScheduleFn:
    """Geometric interpolation between two positive values."""

    def fn(step):
        frac = min(1.0, max(0.0, (step - begin_step) / max(1, end_step - begin_step)))
        return float(begin_value * (end_value / begin_value) ** frac)

    return fn


def inverse_sqrt(*, warmup_steps: int) -> ScheduleFn:
    """``1/sqrt(max(step, warmup_steps))``."""
    return lambda step: float(1.0 / math.sqrt(max(step, warmup_steps)))


def cosine_decay_schedule(*, init_value: float, decay_steps: int, alpha: float = 0.0) -> ScheduleFn:
    def fn(step):
        frac = min(1.0, max(0.0, step / max(1, decay_steps)))
        cos = 0.5 * (1 + math.cos(math.pi * frac))
        return float(init_value * ((1 - alpha) * cos + alpha))

    return fn


def stepwise(*, sub: Sequence[Schedule], start_step: Sequence[int]) -> ScheduleFn:
    """Piecewise schedule: ``sub[i]`` is active from ``start_step[i-1]`` (``sub[0]`` from 0),
    each evaluated on the *global* step."""
    if len(sub) != len(start_step) + 1:
        raise ValueError("len(sub) must be len(start_step) + 1")
    if list(start_step) != sorted(start_step) or any(s <= 0 for s in start_step):
        raise ValueError(f"start_step must be positive and increasing: {start_step}")
    fns = [as_schedule_fn(s) for s in sub]

    def fn(step):
        idx = sum(1 for s in start_step if step >= s)
        return fns[idx](step)

    return fn


def segment_wise(*, segments: Sequence[Schedule], segment_steps: Sequence[int]) -> ScheduleFn:
    """Concatenation of schedules, each evaluated on the step *relative to its own start*;
    ``segment_steps[i]`` is the length of segment ``i`` (the last segment is unbounded)."""
    if len(segments) != len(segment_steps) + 1:
        raise ValueError("len(segments) must be len(segment_steps) + 1")
    fns = [as_schedule_fn(s) for s in segments]
    starts = [0]
    for n in segment_steps:
        starts.append(starts[-1] + n)

    def fn(step):
        idx = 0
        for i, st in enumerate(starts):
            if step >= st:
                idx = i
        return fns[idx](step - starts[idx])

    return fn


def adafactor(*, scale: float = 1.0, warmup_steps: int = 10_000, decay_power: float = -0.5,
              step_offset: int = 0) -> ScheduleFn:
    """Linear warm-up then ``step**decay_power`` decay, continuous at ``warmup_steps``."""

    def fn(step):
        step = max(step - step_offset, 0)
        warm = min(step / max(1, warmup_steps), 1.0)
        return float(scale * warm * max(step, warmup_steps) ** decay_power)

    return fn


def adafactor_decay_rate(c: float = 0.8, step_offset: int = 0) -> ScheduleFn:
    """Second-moment decay of Adafactor: ``1 - (step - step_offset) ** -c`` (0 at the first step)."""

    def fn(step):
        t = float(step) - step_offset
        return 1.0 - t ** (-c) if t > 0 else 0.0

    return fn


def cosine_with_linear_warmup(*, peak_lr: float, warmup_steps: int = 500, max_step: int,
                              begin_value: float = 0.0, alpha: float = 0.0,
                              decay_begin_step: Optional[int] = None) -> ScheduleFn:
    """Linear ``begin_value -> peak_lr`` over ``warmup_steps``, [optional plateau until
    ``decay_begin_step``], then cosine decay to ``alpha * peak_lr`` at ``max_step``."""
    if decay_begin_step is not None and decay_begin_step < warmup_steps:
        raise ValueError("decay_begin_step must be >= warmup_steps")
    segments = [polynomial(begin_value=begin_value, end_value=peak_lr, end_step=warmup_steps)]
    steps = [warmup_steps]
    begin_decay = warmup_steps
    if decay_begin_step is not None and decay_begin_step > warmup_steps:
        segments.append(constant_schedule(peak_lr))
        steps.append(decay_begin_step - warmup_steps)
        begin_decay = decay_begin_step
    segments.append(cosine_decay_schedule(init_value=peak_lr, decay_steps=max_step - begin_decay, alpha=alpha))
    return segment_wise(segments=segments, segment_steps=steps)


def warmup_stable_decay(*, peak_lr: float, max_step: int, warmup_steps: int = 500,
                        decay_steps: Optional[int] = None, begin_value: float = 0.0,
                        end_value: float = 0.0, decay_ratio: float = 0.1) -> ScheduleFn:
    """Linear warm-up, constant plateau, linear decay over the last ``decay_steps``."""
    if decay_steps is None:
        decay_steps = int(max_step * decay_ratio)
    stable = max_step - warmup_steps - decay_steps
    if stable < 0:
        raise ValueError("warmup_steps + decay_steps exceeds max_step")
    return segment_wise(
        segments=[
            polynomial(begin_value=begin_value, end_value=peak_lr, end_step=warmup_steps),
            constant_schedule(peak_lr),
            polynomial(begin_value=peak_lr, end_value=end_value, end_step=decay_steps),
        ],
        segment_steps=[warmup_steps, stable],
    )


def constant_with_linear_warmup(*, peak_lr: float, warmup_steps: int = 500, begin_value: float = 0.0) -> ScheduleFn:
    return segment_wise(
        segments=[
            polynomial(begin_value=begin_value, end_value=peak_lr, end_step=warmup_steps),
            constant_schedule(peak_lr),
        ],
        segment_steps=[warmup_steps],
    )


def linear_schedule_with_warmup(*, peak_lr: float, max_step: int, warmup_steps: int = 500,
                                begin_value: float = 0.0, end_value: float = 0.0) -> ScheduleFn:
    return segment_wise(
        segments=[
            polynomial(begin_value=begin_value, end_value=peak_lr, end_step=warmup_steps),
            polynomial(begin_value=peak_lr, end_value=end_value, end_step=max_step - warmup_steps),
        ],
        segment_steps=[warmup_steps],
    )


def ema_schedule(decay: float = 0.9999, *, warmup_steps: int = 1) -> ScheduleFn:
    """EMA decay ramp ``min(decay, (1 + step) / (warmup_steps + step))``."""
    return lambda step: float(min(decay, (1 + step) / (warmup_steps + step)))
