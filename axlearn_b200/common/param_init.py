"""Parameter initialisers.

``FanAxes`` names which dims of a weight are fan-in / fan-out / batch; ``WeightInitializer``
is variance scaling over those fans; ``DefaultInitializer`` picks an initialiser by regex on
the parameter name (bias → 0, scale → 1, weight → Xavier uniform unless overridden).

Parity targets in the reference (axlearn/common/param_init.py): ``FanAxes`` (:24),
``ConstantInitializer`` (:178), ``GaussianInitializer`` (:209), ``WeightInitializer``
(:283-372), ``DefaultInitializer`` (:375-427), ``PerGroupInitializer`` (:442).  The
``debug_string`` formats are kept so that golden "init" listings stay comparable.

Tensors are drawn directly on the target device from a generator seeded by the host-side
key, one parameter (or one layer slice of a stacked parameter) at a time, so no full-size
host copy of a model is ever made.
"""

from __future__ import annotations

import math
import re
from typing import NamedTuple, Optional, Sequence, Union

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import (
    REQUIRED,
    Configurable,
    InstantiableConfig,
    Required,
    config_class,
)

PARAM_REGEXP_WEIGHT = ".*weight$"
PARAM_REGEXP_BIAS = ".*bias$"
PARAM_REGEXP_SCALE = ".*scale$"

Shape = Sequence[int]
AxisType = Union[int, Sequence[int]]


class FanAxes(NamedTuple):
    """Which axes count as inputs, outputs, and batch (excluded from both fans)."""

    in_axis: AxisType
    out_axis: AxisType
    batch_axis: AxisType = ()

    __config_value__ = True


def _as_tuple(a: AxisType) -> tuple[int, ...]:
    if isinstance(a, int):
        return (a,)
    return tuple(a)


def compute_fans(shape: Shape, axes: FanAxes) -> tuple[float, float]:
    """``(fan_in, fan_out)`` with the receptive-field convention: every dim that is neither
    in, out nor batch multiplies both fans."""
    nd = len(shape)
    norm = lambda ax: tuple(a % nd for a in _as_tuple(ax))
    in_ax, out_ax, batch_ax = norm(axes.in_axis), norm(axes.out_axis), norm(axes.batch_axis)
    in_size = math.prod(shape[a] for a in in_ax)
    out_size = math.prod(shape[a] for a in out_ax)
    batch_size = math.prod(shape[a] for a in batch_ax)
    total = math.prod(shape)
    receptive = total / max(1, in_size * out_size * batch_size)
    return in_size * receptive, out_size * receptive


class Initializer(Configurable):
    """Base class: ``initialize(name, prng_key=, shape=, dtype=, axes=, device=)``."""

    @config_class
    class Config(Configurable.Config):
        pass

    def initialize(
        self,
        name: str,
        *,
        prng_key: torch.Tensor,
        shape: Shape,
        dtype: torch.dtype,
        axes: Optional[FanAxes] = None,
        device="cpu",
    ) -> torch.Tensor:
        raise NotImplementedError(type(self))

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        raise NotImplementedError(type(self))


class ConstantInitializer(Initializer):
    @config_class
    class Config(Initializer.Config):
        value: Required[float] = REQUIRED

    def initialize(self, name, *, prng_key, shape, dtype, axes=None, device="cpu"):
        return torch.full(tuple(shape), self._config.value, dtype=dtype, device=device)

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        return f"constant({self._config.value})"


def constant_initializer(value: float):
    return ConstantInitializer.default_config().set(value=value)


class GaussianInitializer(Initializer):
    @config_class
    class Config(Initializer.Config):
        std: Required[float] = REQUIRED

    def initialize(self, name, *, prng_key, shape, dtype, axes=None, device="cpu"):
        return prng.normal(prng_key, shape, dtype=dtype, device=device, std=self._config.std)

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        return f"normal(0, {self._config.std}^2)"


def gaussian_initializer(std: float):
    return GaussianInitializer.default_config().set(std=std)


class WeightInitializer(Initializer):
    """Variance scaling: ``var = scale / fan`` with ``fan`` in {fan_in, fan_out, fan_avg};
    with ``fan=None`` the scale is the half-range (uniform) or std (normal) directly.
    The default (uniform, fan_avg, scale 1) is Xavier/Glorot uniform."""

    @config_class
    class Config(Initializer.Config):
        scale: float = 1.0
        fan: Optional[str] = "fan_avg"
        distribution: str = "uniform"

    def initialize(self, name, *, prng_key, shape, dtype, axes=None, device="cpu"):
        cfg = self._config
        if cfg.fan is not None:
            if axes is None:
                raise NotImplementedError(f"axes must be provided: {name}")
            fan_in, fan_out = compute_fans(shape, axes)
            if cfg.fan == "fan_in":
                fan = fan_in
            elif cfg.fan == "fan_out":
                fan = fan_out
            elif cfg.fan == "fan_avg":
                fan = (fan_in + fan_out) / 2
            else:
                raise NotImplementedError(f"Unsupported fan {cfg.fan}")
            var = cfg.scale / max(1.0, fan)
            if cfg.distribution == "uniform":
                lim = math.sqrt(3.0 * var)
                return prng.uniform(
                    prng_key, shape, dtype=dtype, device=device, minval=-lim, maxval=lim
                )
            if cfg.distribution == "normal":
                return prng.normal(prng_key, shape, dtype=dtype, device=device, std=math.sqrt(var))
            if cfg.distribution == "truncated_normal":
                return prng.truncated_normal(
                    prng_key, shape, dtype=dtype, device=device, std=math.sqrt(var)
                )
            raise NotImplementedError(f"Unsupported distribution {cfg.distribution}")
        if cfg.distribution == "uniform":
            return prng.uniform(
                prng_key, shape, dtype=dtype, device=device, minval=-cfg.scale, maxval=cfg.scale
            )
        if cfg.distribution == "normal":
            return prng.normal(prng_key, shape, dtype=dtype, device=device, std=cfg.scale)
        if cfg.distribution == "truncated_normal":
            return prng.truncated_normal(prng_key, shape, dtype=dtype, device=device, std=cfg.scale)
        raise NotImplementedError(f"Unsupported fan {cfg.fan} / distribution {cfg.distribution}")

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        cfg = self._config
        if cfg.fan is not None:
            if cfg.distribution == "uniform":
                return (
                    f"uniform(-sqrt({3 * cfg.scale} / {cfg.fan}), "
                    f"sqrt({3 * cfg.scale} / {cfg.fan})), shape={shape}, axes={axes}"
                )
            if cfg.distribution == "normal":
                return f"normal(0, {cfg.scale} / {cfg.fan}), shape={shape}, axes={axes}"
            if cfg.distribution == "truncated_normal":
                return (
                    f"truncated_normal(-2, 2) * sqrt({cfg.scale} / {cfg.fan}) / 0.88, "
                    f"shape={shape}, axes={axes}"
                )
            raise NotImplementedError(cfg.distribution)
        if cfg.distribution == "uniform":
            return f"uniform({-cfg.scale}, {cfg.scale})"
        if cfg.distribution == "normal":
            return f"normal(0, {cfg.scale}^2)"
        if cfg.distribution == "truncated_normal":
            return f"truncated_normal(-2, 2) * {cfg.scale} / 0.88"
        raise NotImplementedError(cfg.distribution)


class DefaultInitializer(Initializer):
    """Chooses an initialiser by the first regex (insertion order) that fully matches the
    parameter name.  User rules are consulted before the built-in bias/scale/weight rules."""

    @config_class
    class Config(Initializer.Config):
        init_by_param_name: dict[str, InstantiableConfig] = {}

    def __init__(self, cfg: "DefaultInitializer.Config"):
        cfg = cfg.clone()
        rules = dict(cfg.init_by_param_name)
        rules.setdefault(PARAM_REGEXP_BIAS, constant_initializer(0.0))
        rules.setdefault(PARAM_REGEXP_SCALE, constant_initializer(1.0))
        rules.setdefault(PARAM_REGEXP_WEIGHT, WeightInitializer.default_config())
        cfg.init_by_param_name = rules
        super().__init__(cfg)
        self._rules = [(re.compile(p), c.instantiate()) for p, c in rules.items()]

    def _pick(self, name: str) -> Initializer:
        for pattern, init in self._rules:
            if pattern.fullmatch(name):
                return init
        raise NotImplementedError(f"Unsupported parameter name ({name})")

    def initialize(self, name, *, prng_key, shape, dtype, axes=None, device="cpu"):
        return self._pick(name).initialize(
            name, prng_key=prng_key, shape=shape, dtype=dtype, axes=axes, device=device
        )

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        return self._pick(name).debug_string(name=name, shape=shape, axes=axes)


class PerGroupInitializer(Initializer):
    """Splits ``axis`` into ``num_groups`` groups and initialises each group separately, so
    that fans are computed per group (grouped convolutions / grouped projections)."""

    @config_class
    class Config(Initializer.Config):
        initializer: Required[InstantiableConfig] = REQUIRED
        num_groups: Required[int] = REQUIRED
        axis: int = -1

    def __init__(self, cfg):
        super().__init__(cfg)
        self._inner = cfg.initializer.instantiate()

    def initialize(self, name, *, prng_key, shape, dtype, axes=None, device="cpu"):
        cfg = self._config
        ax = cfg.axis % len(shape)
        if shape[ax] % cfg.num_groups:
            raise ValueError(f"dim {shape[ax]} not divisible by num_groups {cfg.num_groups}")
        gshape = list(shape)
        gshape[ax] //= cfg.num_groups
        keys = prng.split(prng_key, cfg.num_groups)
        parts = [
            self._inner.initialize(
                name, prng_key=k, shape=gshape, dtype=dtype, axes=axes, device=device
            )
            for k in keys
        ]
        return torch.cat(parts, dim=ax)

    def debug_string(self, name=None, shape=None, axes=None) -> str:
        cfg = self._config
        return (
            f"per_group(num_groups={cfg.num_groups}, axis={cfg.axis}, "
            f"{self._inner.debug_string(name=name, shape=shape, axes=axes)})"
        )
