"""Per-token activation-gradient monitoring and clipping between transformer blocks.

Reference: axlearn/common/gradient_monitor.py (clip functions :42-117, position encoding :120-134,
``GradientMonitorAndClipLayer`` :259-332, ``create_monitored_layer_class`` :335-367,
``convert_to_monitored_layer_config`` :370-400, learner modifier :403-431).

A monitored layer's output passes through an identity whose backward sees dL/dy.  The backward
zeroes the tokens with the largest gradient norms (or only measures percentiles) and hands the
statistics back as the "gradient" of the layer's ``stats`` parameter; a sub-learner with
``replace_with_updates`` stores them as the parameter's next value, and the next forward pass
writes them to the summaries.  Here the identity is a ``torch.autograd.Function``.
"""

from __future__ import annotations

import functools
from typing import Any, Callable, Optional, Sequence

import torch

from axlearn_b200.common import learner, optimizers
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import InstantiableConfig, config_class, config_for_function
from axlearn_b200.common.param_init import ConstantInitializer
from axlearn_b200.common.utils import flatten_items, unflatten_items

Tensor = torch.Tensor

DEFAULT_PERCENTILES = (50, 99.9, 99.99, 99.999)
# "" = the output itself is the tensor (feed-forward); "data" = attention's output field.
GRADIENT_CLIPPING_PATHS = ("", "data")


def _token_norms(g: Tensor) -> Tensor:
    return torch.linalg.vector_norm(g.float(), dim=-1)


def compute_grad_percentile_no_clip_fn(stats_arr: Sequence[float] = DEFAULT_PERCENTILES):
    """Measures percentiles of the per-token gradient norm; the gradient passes unchanged."""
    q = torch.tensor([p / 100.0 for p in stats_arr], dtype=torch.float64)

    def fn(g: Tensor):
        norms = _token_norms(g).reshape(-1).double()
        return g, torch.quantile(norms, q.to(norms.device)).float()

    return fn


def encode_int32_to_bf16_bytes(x: Tensor) -> Tensor:
    """``[k]`` int32 -> ``[4, k]`` bf16 of base-256 digits (least significant first): token
    positions stay exact in a bf16 training step."""
    ux = x.to(torch.int64) & 0xFFFFFFFF
    return torch.stack([((ux >> s) & 0xFF).to(torch.bfloat16) for s in (0, 8, 16, 24)], dim=0)


def decode_bf16_bytes_to_int32(d: Tensor) -> Tensor:
    v = sum(d[i].to(torch.int64) << (8 * i) for i in range(4))
    return torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32)


def top_k_clip_fn(k: int = 4, method: str = "topk", log_pos: bool = False):
    """Zeroes the gradient of the ``k`` tokens of the batch with the largest gradient norm.

    ``method``: "approx" and "topk" both run an exact top-k here (there is no approximate
    variant worth having on a GPU at these sizes); "sort" sorts.  "approx" removes exactly the
    chosen ids, the other two remove every token at or above the k-th norm, as the reference
    does.  Statistics: the k norms in descending order, plus the encoded positions when
    ``log_pos``.
    """
    if method not in ("approx", "topk", "sort"):
        raise ValueError(f"unknown method {method}")

    def fn(g: Tensor):
        norms = _token_norms(g)
        flat = norms.reshape(-1)
        if not 1 <= k < flat.numel():
            raise ValueError("k must be >= 1 and < token count")
        if method == "sort":
            ids = torch.argsort(flat, descending=True)[:k]
            top = flat[ids]
        else:
            top, ids = torch.topk(flat, k)
        if method == "approx":
            keep = torch.ones_like(flat, dtype=torch.bool)
            keep[ids] = False
            keep = keep.reshape(norms.shape)
        else:
            keep = norms < top[-1]
        clipped = torch.where(keep.unsqueeze(-1), g, torch.zeros((), dtype=g.dtype, device=g.device))
        if log_pos:
            stats = torch.cat([top[None, :].to(torch.bfloat16), encode_int32_to_bf16_bytes(ids)], dim=0).float()
        else:
            stats = top
        return clipped, stats

    return fn


def gradient_clipping_impl(g: Any, *, clip_fn: Callable, prev_stats: Optional[Tensor] = None,
                           supported_paths: Sequence[str] = GRADIENT_CLIPPING_PATHS):
    """Applies ``clip_fn`` to the one leaf of ``g`` whose path is in ``supported_paths``."""
    del prev_stats
    if isinstance(g, Tensor):
        items = [("", g)]
    else:
        items = list(flatten_items(g, is_leaf=lambda x: x is None or isinstance(x, Tensor)))
    out, stats = [], []
    for path, leaf in items:
        if path in set(supported_paths) and leaf is not None:
            if not isinstance(leaf, Tensor):
                raise TypeError("monitoring applies to plain tensors")
            leaf, s = clip_fn(leaf)
            stats.append(s)
        out.append((path, leaf))
    if len(stats) != 1:
        raise ValueError(f"expected exactly one monitored tensor per layer, got {len(stats)}")
    clipped = out[0][1] if isinstance(g, Tensor) else unflatten_items(out)
    return clipped, stats[0]


class _ClipGradient(torch.autograd.Function):
    """Identity forward; the backward clips dL/dy and returns the statistics as d/d(stats)."""

    @staticmethod
    def forward(ctx, x, prev_stats, clip_fn):  # pylint: disable=arguments-differ
        ctx.clip_fn = clip_fn
        ctx.stats_meta = (prev_stats.shape, prev_stats.dtype)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):  # pylint: disable=arguments-differ
        clipped, stats = ctx.clip_fn(g)
        shape, dtype = ctx.stats_meta
        return clipped, stats.reshape(shape).to(dtype), None


def _top_norms(stats: Tensor) -> Tensor:
    return stats[0] if stats.ndim > 1 else stats


def default_stats_logging_fn(log_pos: bool = False):
    """``fn(layer, stats)``: histogram of the top norms; with ``log_pos`` also the largest norm,
    the clip threshold and the decoded positions."""

    def fn(layer: "GradientMonitorAndClipLayer", stats: Tensor) -> None:
        top = _top_norms(stats)
        if log_pos:
            if stats.ndim < 2:
                raise ValueError("log_pos=True but the statistics carry no positions; "
                                 "set clip_fn.log_pos and stats_shape=(5, k)")
            layer.add_summary("max_norm", top[0])
            layer.add_summary("clip_threshold", top[-1])
            layer.add_summary("clipped_token_pos", decode_bf16_bytes_to_int32(stats[1:]))
        layer.add_summary("top_norms_hist", top)

    return fn


class GradientMonitorAndClipLayer(BaseLayer):
    """Child of a monitored layer: ``y = monitor(y)`` is the identity with a clipping backward."""

    @config_class
    class Config(BaseLayer.Config):
        supported_paths: Sequence[str] = GRADIENT_CLIPPING_PATHS
        stats_shape: tuple = (4,)
        clip_fn: InstantiableConfig = config_for_function(top_k_clip_fn)
        stats_log_fn: InstantiableConfig = config_for_function(default_stats_logging_fn)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        log_cfg = cfg.stats_log_fn
        if "log_pos" in cfg.clip_fn.keys() and "log_pos" in log_cfg.keys():
            log_cfg = log_cfg.clone(log_pos=cfg.clip_fn.log_pos)
        self._clip_fn = cfg.clip_fn.instantiate()
        self._stats_log_fn = functools.partial(log_cfg.instantiate(), self)

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"stats": ParameterSpec(
            shape=tuple(cfg.stats_shape), mesh_axes=(None,) * len(cfg.stats_shape),
            initializer=ConstantInitializer.default_config().set(value=0.0).instantiate())}

    def forward(self, x: Any) -> Any:
        cfg = self._config
        prev = self.parameters["stats"]
        self._stats_log_fn(prev.detach())  # statistics of the previous backward pass
        if isinstance(x, Tensor):
            if "" not in cfg.supported_paths:
                raise ValueError('a tensor output needs "" in supported_paths')
            return _ClipGradient.apply(x, prev, self._clip_fn)
        hit = 0
        out = []
        for path, leaf in flatten_items(x, is_leaf=lambda v: v is None or isinstance(v, Tensor)):
            if path in cfg.supported_paths and isinstance(leaf, Tensor):
                leaf = _ClipGradient.apply(leaf, prev, self._clip_fn)
                hit += 1
            out.append((path, leaf))
        if hit != 1:
            raise ValueError(f"expected exactly one monitored tensor per layer, got {hit}")
        rebuilt = unflatten_items(out)
        if hasattr(x, "_replace"):  # named tuples keep their type
            return type(x)(**rebuilt)
        return rebuilt


@functools.lru_cache(maxsize=None)
def create_monitored_layer_class(base_class: type) -> type:
    """``Monitored<Base>``: the base layer with a ``gradient_monitor`` child on its output."""

    class MonitoredLayer(base_class):
        @config_class
        class Config(base_class.Config):
            gradient_monitor: Optional[InstantiableConfig] = GradientMonitorAndClipLayer.default_config()

        def __init__(self, cfg, *, parent=None):
            super().__init__(cfg, parent=parent)
            if cfg.gradient_monitor is not None:
                self._add_child("gradient_monitor", cfg.gradient_monitor)

        def forward(self, *args, **kwargs):
            y = super().forward(*args, **kwargs)
            if self._config.gradient_monitor is not None:
                y = self.gradient_monitor(y)
            return y

    MonitoredLayer.__name__ = MonitoredLayer.__qualname__ = f"Monitored{base_class.__name__}"
    return MonitoredLayer


def convert_to_monitored_layer_config(cfg: InstantiableConfig,
                                      gradient_monitor_cfg: Optional[InstantiableConfig] = None):
    """A config of ``Monitored<cfg.klass>`` with every field of ``cfg`` carried over."""
    monitored = create_monitored_layer_class(cfg.klass).default_config()
    for name, value in cfg.items():
        if name != "klass":
            setattr(monitored, name, value)
    return monitored.set(gradient_monitor=gradient_monitor_cfg or GradientMonitorAndClipLayer.default_config())


def gradient_monitoring_learner_cfg_modifier(learner_cfg: InstantiableConfig) -> InstantiableConfig:
    """Wraps a learner so that ``.../gradient_monitor/stats`` takes its gradient as its value."""
    stats_learner = learner.Learner.default_config().set(
        optimizer=config_for_function(optimizers.replace_with_updates))
    ema_decay = learner_cfg.ema.decay
    learner_cfg.ema.decay = None
    cfg = learner.CompositeLearner.default_config().set(
        learners={"inner": learner_cfg, "gradient_monitor_stats": stats_learner},
        rules=[(".*gradient_monitor/stats", "gradient_monitor_stats"), (".*", "inner")])
    cfg.ema.decay = ema_decay
    return cfg
