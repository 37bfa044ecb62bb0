"""Basic layers: norms, Linear, Embedding, Dropout and friends.

Parity targets in the reference (axlearn/common/layers.py): ``get_activation_fn`` (:72),
``RedirectToSharedModule`` (:94), ``Dropout`` (:169), ``LayerNorm`` (:336), ``RMSNorm``
(:403), ``L2Norm`` (:425), ``GroupNorm`` (:527), ``BatchNorm`` (:650), ``Linear`` (:715),
``Embedding`` (:836), ``StochasticDepth`` (:1221), ``SqueezeExcitation`` (:1312),
``MovingAverage`` (:1527) and the recursive config setters (:239, :264, :1284, :1298).

Sharding: a parameter's ``param_partition_spec`` names mesh axes per dim.  Axes other than
``model`` shard storage only (FSDP): the layer gathers over them right before use and the
gradient is reduce-scattered back.  ``model`` shards the computation (tensor parallelism):
``Linear`` with ``model`` on its output dim is column-parallel (no forward collective, input
gradient summed over ``model``); with ``model`` on its input dim it is row-parallel (partial
outputs summed over ``model``).
"""

from __future__ import annotations

import math
from typing import Any, Callable, Optional, Sequence, Union

import torch
import torch.nn.functional as F

from axlearn_b200 import ops
from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer, FactorizationSpec, ParameterSpec
from axlearn_b200.common.config import (
    REQUIRED,
    ConfigBase,
    InstantiableConfig,
    Required,
    config_class,
)
from axlearn_b200.common.module import Module, nowrap
from axlearn_b200.common.param_init import FanAxes, WeightInitializer, constant_initializer
from axlearn_b200.parallel import collectives as coll

Tensor = torch.Tensor


def quick_gelu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(1.702 * x)


def squared_relu(x: Tensor) -> Tensor:
    return torch.square(F.relu(x))


_ACTIVATIONS: dict[str, Callable[[Tensor], Tensor]] = {
    "linear": lambda x: x,
    "quick_gelu": quick_gelu,
    "exact_gelu": lambda x: F.gelu(x, approximate="none"),
    "squared_relu": squared_relu,
    "nn.relu": F.relu,
    "nn.relu6": F.relu6,
    "nn.silu": F.silu,
    "nn.swish": F.silu,
    "nn.gelu": lambda x: F.gelu(x, approximate="tanh"),
    "nn.sigmoid": torch.sigmoid,
    "nn.tanh": torch.tanh,
    "nn.softplus": F.softplus,
    "nn.elu": F.elu,
    "nn.leaky_relu": F.leaky_relu,
    "nn.hard_swish": F.hardswish,
    "nn.hard_sigmoid": F.hardsigmoid,
    "nn.hard_tanh": F.hardtanh,
    "jnp.tanh": torch.tanh,
}


def get_activation_fn(name: str) -> Callable[[Tensor], Tensor]:
    """Maps the reference's activation names (``"nn.silu"``, ``"linear"``, ...) to
    callables."""
    if name not in _ACTIVATIONS:
        raise ValueError(f"Unsupported activation function {name}")
    return _ACTIVATIONS[name]


class RedirectToSharedModule(BaseLayer):
    """Forwards method calls to a module shared by an ancestor (weight tying)."""

    @config_class
    class Config(BaseLayer.Config):
        shared_module: Required[str] = REQUIRED
        # {method on this layer: method on the shared module}; default = same name.
        method_map: dict[str, str] = {}

    def __getattr__(self, name: str) -> Any:
        if name.startswith("_"):
            raise AttributeError(name)
        cfg = self.__dict__.get("_config")
        if cfg is None:
            raise AttributeError(name)
        target = self.get_shared_module(cfg.shared_module)
        return getattr(target, cfg.method_map.get(name, name))

    def forward(self, *args, **kwargs):
        cfg = self._config
        target = self.get_shared_module(cfg.shared_module)
        return getattr(target, cfg.method_map.get("forward", "forward"))(*args, **kwargs)


class Dropout(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        rate: Optional[float] = None

    def forward(self, x: Tensor) -> Tensor:
        rate = self._config.rate
        if not self.is_training or not rate:
            return x
        if not 0 < rate < 1:
            raise ValueError(f"Dropout rate must be in (0, 1): {rate}")
        keep = prng.bernoulli(self.prng_key, 1 - rate, x.shape, device=x.device)
        return torch.where(keep, x / (1 - rate), torch.zeros_like(x))


class DropToken(BaseLayer):
    """Randomly keeps ``num_tokens * (1 - rate)`` tokens per example during training."""

    @config_class
    class Config(BaseLayer.Config):
        num_cls_tokens: int = 0
        rate: float = 0.0

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        if not self.is_training or cfg.rate <= 0:
            return x
        b, n, _ = x.shape
        body = n - cfg.num_cls_tokens
        keep = int(body * (1 - cfg.rate))
        noise = prng.uniform(self.prng_key, (b, body), device=x.device)
        idx = noise.argsort(dim=1)[:, :keep].sort(dim=1).values + cfg.num_cls_tokens
        if cfg.num_cls_tokens:
            cls = torch.arange(cfg.num_cls_tokens, device=x.device).expand(b, -1)
            idx = torch.cat([cls, idx], dim=1)
        return torch.gather(x, 1, idx[:, :, None].expand(-1, -1, x.shape[-1]))


class BaseNormalizationLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        raise NotImplementedError(type(self))


class LayerNormStateless(BaseNormalizationLayer):
    @config_class
    class Config(BaseNormalizationLayer.Config):
        eps: float = 1e-8
        forward_dtype: Optional[torch.dtype] = torch.float32

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        dt = x.dtype
        if cfg.forward_dtype is not None:
            x = x.to(cfg.forward_dtype)
        mean = x.mean(-1, keepdim=True)
        x = x - mean
        var = (x * x).mean(-1, keepdim=True)
        return (x * torch.rsqrt(var + cfg.eps)).to(dt)


class LayerNorm(LayerNormStateless):
    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {
            "scale": ParameterSpec(shape=(cfg.input_dim,), mesh_axes=(None,)),
            "bias": ParameterSpec(shape=(cfg.input_dim,), mesh_axes=(None,)),
        }

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        y = super().forward(x)
        return y * self.parameters["scale"].to(y.dtype) + self.parameters["bias"].to(y.dtype)


class RMSNormStateless(BaseNormalizationLayer):
    @config_class
    class Config(BaseNormalizationLayer.Config):
        eps: float = 1e-8
        forward_dtype: Optional[torch.dtype] = torch.float32
        input_partition_spec: Optional[Sequence[Any]] = None
        output_partition_spec: Optional[Sequence[Any]] = None

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        ones = torch.ones(x.shape[-1], dtype=x.dtype, device=x.device)
        return ops.rms_norm(x, ones, cfg.eps, upcast=cfg.forward_dtype == torch.float32)


class RMSNorm(RMSNormStateless):
    """``x * rsqrt(mean(x^2) + eps) * scale``; statistics in ``forward_dtype`` (fp32 by
    default; ``None`` = the activation dtype)."""

    def _create_layer_parameter_specs(self):
        return {"scale": ParameterSpec(shape=(self._config.input_dim,), mesh_axes=(None,))}

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        return ops.rms_norm(
            x, self.parameters["scale"], cfg.eps, upcast=cfg.forward_dtype == torch.float32
        )

    def forward_keep_input(self, x: Tensor) -> tuple[Tensor, Tensor]:
        """``(norm(x), x)`` for a pre-norm block: use the second output for the residual branch
        and its gradient is added inside the norm's backward pass."""
        cfg = self._config
        return ops.rms_norm_keep_input(x, self.parameters["scale"], cfg.eps, upcast=cfg.forward_dtype == torch.float32)

    def forward_add(self, x: Tensor, residual: Tensor) -> tuple[Tensor, Tensor]:
        """``(x + residual, norm(x + residual))`` in one pass."""
        cfg = self._config
        return ops.add_rms_norm(x, residual, self.parameters["scale"], cfg.eps,
                                upcast=cfg.forward_dtype == torch.float32)


class L2Norm(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        eps: float = 1e-8

    def forward(self, x: Tensor) -> Tensor:
        return x * torch.rsqrt((x.float() ** 2).sum(-1, keepdim=True) + self._config.eps).to(x.dtype)


class GroupNorm(BaseNormalizationLayer):
    """Normalises over (spatial..., channels-in-group); input ``[B, ..., C]``."""

    @config_class
    class Config(BaseNormalizationLayer.Config):
        num_groups: Required[int] = REQUIRED
        eps: float = 1e-8
        forward_dtype: Optional[torch.dtype] = torch.float32

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {
            "scale": ParameterSpec(shape=(cfg.input_dim,), mesh_axes=(None,)),
            "bias": ParameterSpec(shape=(cfg.input_dim,), mesh_axes=(None,)),
        }

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        dt = x.dtype
        if cfg.forward_dtype is not None:
            x = x.to(cfg.forward_dtype)
        b, c = x.shape[0], x.shape[-1]
        g = cfg.num_groups
        xg = x.reshape(b, -1, g, c // g)
        if paddings is None:
            mean = xg.mean(dim=(1, 3), keepdim=True)
            var = ((xg - mean) ** 2).mean(dim=(1, 3), keepdim=True)
        else:
            w = (1 - paddings.to(x.dtype)).reshape(b, -1, 1, 1)
            cnt = (w.sum(dim=1, keepdim=True) * (c // g)).clamp_min(1.0)
            mean = (xg * w).sum(dim=(1, 3), keepdim=True) / cnt
            var = (((xg - mean) ** 2) * w).sum(dim=(1, 3), keepdim=True) / cnt
        y = ((xg - mean) * torch.rsqrt(var + cfg.eps)).reshape(x.shape).to(dt)
        y = y * self.parameters["scale"].to(dt) + self.parameters["bias"].to(dt)
        if paddings is not None:
            y = y * (1 - paddings.to(dt)).reshape(paddings.shape + (1,) * (y.dim() - paddings.dim()))
        return y


class BatchNorm(BaseNormalizationLayer):
    """Batch norm over all dims but the last; moving statistics are non-trainable state
    updated through ``add_state_update``."""

    @config_class
    class Config(BaseNormalizationLayer.Config):
        decay: float = 0.999
        eps: float = 1e-3

    def _create_layer_parameter_specs(self):
        d = self._config.input_dim
        return {
            "scale": ParameterSpec(shape=(d,), mesh_axes=(None,)),
            "bias": ParameterSpec(shape=(d,), mesh_axes=(None,)),
            "moving_mean": ParameterSpec(
                shape=(d,), dtype=torch.float32, mesh_axes=(None,),
                initializer=constant_initializer(0.0), weight_decay_scale=0,
            ),
            "moving_variance": ParameterSpec(
                shape=(d,), dtype=torch.float32, mesh_axes=(None,),
                initializer=constant_initializer(1.0), weight_decay_scale=0,
            ),
        }

    def forward(self, x: Tensor, *, paddings: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        p = self.parameters
        if self.is_training:
            red = tuple(range(x.dim() - 1))
            xf = x.float()
            if paddings is not None:
                # Statistics over the unpadded positions only.
                w = (1 - paddings.float()).reshape(paddings.shape + (1,) * (x.dim() - paddings.dim()))
                n = (w.sum() * (xf[..., 0].numel() / max(1, w.numel()))).clamp_min(1.0)
                mean = (xf * w).sum(dim=red) / n
                var = (((xf - mean) ** 2) * w).sum(dim=red) / n
                live_mean, live_var = mean, var
            else:
                mean = xf.mean(dim=red)
                var = ((xf - mean) ** 2).mean(dim=red)
                live_mean, live_var = mean, var
            mean = coll.all_reduce_scalar(mean, ("data", "expert", "fsdp")) / coll.axis_size(("data", "expert", "fsdp"))
            var = coll.all_reduce_scalar(var, ("data", "expert", "fsdp")) / coll.axis_size(("data", "expert", "fsdp"))
            d = cfg.decay
            self.add_state_update("moving_mean", (d * p["moving_mean"] + (1 - d) * mean).detach())
            self.add_state_update("moving_variance", (d * p["moving_variance"] + (1 - d) * var).detach())
            y = (xf - live_mean) * torch.rsqrt(live_var + cfg.eps)
        else:
            y = (x.float() - p["moving_mean"]) * torch.rsqrt(p["moving_variance"] + cfg.eps)
        return (y * p["scale"].float() + p["bias"].float()).to(x.dtype)


# ------------------------------------------------------------------------------------------
# Linear / Embedding.
# ------------------------------------------------------------------------------------------


def _spec_entry(spec: Optional[Sequence[Any]], dim: int) -> Any:
    if spec is None:
        return None
    return spec[dim]


class DenseGeneralBaseLayer(BaseLayer):
    """Base of layers whose main op is a contraction; an optional ``quantized_dot_general``
    child config replaces the plain matmul (fp8)."""

    @config_class
    class Config(BaseLayer.Config):
        quantized_dot_general: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.quantized_dot_general is not None:
            self._add_child("quantized_dot_general", cfg.quantized_dot_general)

    @nowrap
    def _plain_matmul(self) -> bool:
        """True when products of this layer are ordinary bf16 GEMMs (no quantised path)."""
        return "quantized_dot_general" not in self._children

    def _matmul(self, x: Tensor, w: Tensor) -> Tensor:
        """``x[..., K] @ w[K, N]`` routed through the quantised path when configured."""
        if "quantized_dot_general" in self._children:
            return self._children["quantized_dot_general"].matmul(x, w)
        return ops.linear(x, w)


class Linear(DenseGeneralBaseLayer):
    """``y = x @ weight (+ bias)``, weight ``[input_dim, output_dim]``."""

    @config_class
    class Config(DenseGeneralBaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        bias: bool = True
        output_partition_spec: Optional[Sequence[Any]] = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.param_partition_spec = (None, "model")
        return cfg

    def _create_layer_parameter_specs(self):
        cfg = self._config
        spec = cfg.param_partition_spec
        params = {
            "weight": ParameterSpec(
                shape=(cfg.input_dim, cfg.output_dim),
                mesh_axes=spec,
                factorization=FactorizationSpec(axes=("row", "col")),
            )
        }
        if cfg.bias:
            params["bias"] = ParameterSpec(
                shape=(cfg.output_dim,), mesh_axes=(_spec_entry(spec, -1),) if spec else None
            )
        return params

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        spec = cfg.param_partition_spec
        w = self.parameters["weight"]
        cshape = coll.compute_shape((cfg.input_dim, cfg.output_dim), spec)
        w = coll.unshard_param(w, spec, compute_shape=cshape)
        col_parallel = coll.has_axis(_spec_entry(spec, 1), "model")
        row_parallel = coll.has_axis(_spec_entry(spec, 0), "model")
        if col_parallel:
            x = coll.tp_enter(x, "model")
        wx = w.to(x.dtype) if w.dtype != x.dtype else w
        y = coll.row_parallel_linear(x, wx, "model") if row_parallel and self._plain_matmul() else None
        if y is None:
            y = self._matmul(x, wx)
            if row_parallel:
                y = coll.tp_exit(y, "model")
        if cfg.bias:
            b = self.parameters["bias"]
            b = coll.unshard_param(b, (_spec_entry(spec, -1),) if spec else None,
                                   compute_shape=(cshape[1],))
            y = y + b.to(y.dtype)
        return y


class UnitNormLinear(Linear):
    """Linear whose weight columns are L2-normalised before use."""

    def forward(self, x: Tensor) -> Tensor:
        w = self.parameters["weight"]
        w = w * torch.rsqrt((w.float() ** 2).sum(0, keepdim=True) + 1e-8).to(w.dtype)
        return ops.linear(x, w.to(x.dtype))


class MultiLinear(BaseLayer):
    """``num_outputs`` parallel projections: weight ``[input_dim, num_outputs, output_dim]``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_outputs: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        bias: bool = True

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = {
            "weight": ParameterSpec(
                shape=(cfg.input_dim, cfg.num_outputs, cfg.output_dim),
                mesh_axes=cfg.param_partition_spec or (None, None, None),
                fan_axes=FanAxes(in_axis=0, out_axis=(1, 2)),
            )
        }
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.num_outputs, cfg.output_dim), mesh_axes=(None, None))
        return params

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        w = self.parameters["weight"].to(x.dtype)
        y = ops.linear(x, w.reshape(cfg.input_dim, -1)).reshape(x.shape[:-1] + (cfg.num_outputs, cfg.output_dim))
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y


class Embedding(BaseLayer):
    """Token embedding ``weight[num_embeddings, dim]``; ``attend`` reuses it as a tied
    output head."""

    @config_class
    class Config(BaseLayer.Config):
        num_embeddings: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        input_partition_spec: Optional[Sequence[Any]] = None
        embedding_partition_spec: Optional[Sequence[Any]] = None
        output_partition_spec: Optional[Sequence[Any]] = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.param_partition_spec = (None, "model")
        # Normal with std 1/sqrt(dim).
        cfg.param_init = None
        return cfg

    def _create_layer_parameter_specs(self):
        cfg = self._config
        init = None
        if cfg.param_init is None:
            from axlearn_b200.common.param_init import DefaultInitializer, PARAM_REGEXP_WEIGHT

            init = DefaultInitializer.default_config().set(
                init_by_param_name={
                    PARAM_REGEXP_WEIGHT: WeightInitializer.default_config().set(
                        fan="fan_out", distribution="normal"
                    )
                }
            )
        return {
            "weight": ParameterSpec(
                shape=(cfg.num_embeddings, cfg.dim),
                mesh_axes=cfg.param_partition_spec,
                initializer=init,
            )
        }

    def _weight(self) -> Tensor:
        cfg = self._config
        spec = cfg.param_partition_spec
        cshape = coll.compute_shape((cfg.num_embeddings, cfg.dim), spec)
        return coll.unshard_param(self.parameters["weight"], spec, compute_shape=cshape)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        w = self._weight()
        y = F.embedding(x.long(), w)
        if coll.has_axis(_spec_entry(cfg.param_partition_spec, 1), "model"):
            # Feature dim is split over "model": assemble full rows.
            y = coll.all_gather(y, "model", dim=-1)
        elif coll.has_axis(_spec_entry(cfg.param_partition_spec, 0), "model"):
            raise NotImplementedError("vocab-parallel embedding lookup")
        return y

    def embeddings(self) -> Tensor:
        """The whole table ``[num_embeddings, dim]``."""
        w = self._weight()
        if coll.has_axis(_spec_entry(self._config.param_partition_spec, 1), "model"):
            w = coll.all_gather(w, "model", dim=1)
        return w

    def attend(self, x: Tensor) -> Tensor:
        """``logits[..., n] = sum_d x[..., d] * weight[n, d]``."""
        w = self._weight()
        if coll.has_axis(_spec_entry(self._config.param_partition_spec, 1), "model"):
            w = coll.all_gather(w, "model", dim=1)
        return ops.linear(x, w.to(x.dtype).t())

    @nowrap
    def embedding_weight_for_loss(self, params: dict) -> Tensor:
        return params["weight"]


class StochasticDepth(BaseLayer):
    """Drops the whole residual branch per example with probability ``rate``."""

    @config_class
    class Config(BaseLayer.Config):
        rate: Optional[float] = None
        mode: str = "row"

    def forward(self, x: Tensor) -> Tensor:
        rate = self._config.rate
        if not self.is_training or not rate:
            return x
        shape = (x.shape[0],) + (1,) * (x.dim() - 1) if self._config.mode == "row" else (1,) * x.dim()
        keep = prng.bernoulli(self.prng_key, 1 - rate, shape, device=x.device)
        return x * keep.to(x.dtype) / (1 - rate)


class SqueezeExcitation(BaseLayer):
    """Channel gating from globally pooled features; input ``[B, H, W, C]``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        se_ratio: float = 0.0
        activation: str = "nn.relu"
        gating: str = "nn.sigmoid"
        num_reduced_filters: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.se_ratio > 0:
            reduced = cfg.num_reduced_filters or max(1, int(cfg.input_dim * cfg.se_ratio))
            self._add_child("reduce", Linear.default_config().set(input_dim=cfg.input_dim, output_dim=reduced))
            self._add_child("expand", Linear.default_config().set(input_dim=reduced, output_dim=cfg.input_dim))

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        if cfg.se_ratio <= 0:
            return x
        pooled = x.mean(dim=(1, 2), keepdim=True)
        h = get_activation_fn(cfg.activation)(self.reduce(pooled))
        return x * get_activation_fn(cfg.gating)(self.expand(h))


class VariationalNoise(BaseLayer):
    """Adds Gaussian noise to activations in training."""

    @config_class
    class Config(BaseLayer.Config):
        vn_std: Optional[float] = None

    def forward(self, x: Tensor) -> Tensor:
        std = self._config.vn_std
        if not self.is_training or not std:
            return x
        return x + prng.normal(self.prng_key, x.shape, dtype=x.dtype, device=x.device, std=std)


class MovingAverage(BaseLayer):
    """Exponential moving average of a (scalar or tensor) statistic kept as state."""

    @config_class
    class Config(BaseLayer.Config):
        shape: Sequence[int] = ()
        min_weight: float = 0.001

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {
            "count": ParameterSpec(shape=(), dtype=torch.int32, mesh_axes=(), initializer=constant_initializer(0), weight_decay_scale=0),
            "value": ParameterSpec(shape=tuple(cfg.shape), dtype=torch.float32, mesh_axes=(None,) * len(cfg.shape), initializer=constant_initializer(0.0), weight_decay_scale=0),
        }

    def forward(self, x: Tensor) -> Tensor:
        p = self.parameters
        count = p["count"] + 1
        w = torch.clamp(1.0 / count.float(), min=self._config.min_weight)
        new = (1 - w) * p["value"] + w * x.detach().float()
        self.add_state_update("count", count)
        self.add_state_update("value", new)
        return new


class MaxPool2D(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        window: tuple[int, int] = (2, 2)
        strides: tuple[int, int] = (1, 1)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        y = F.max_pool2d(x.permute(0, 3, 1, 2), cfg.window, cfg.strides)
        return y.permute(0, 2, 3, 1)


# ------------------------------------------------------------------------------------------
# Recursive config setters.
# ------------------------------------------------------------------------------------------


def _visit_configs(cfg: ConfigBase, fn: Callable[[ConfigBase], None]) -> None:
    fn(cfg)
    for _, v in cfg.items():
        _visit_value(v, fn)


def _visit_value(v: Any, fn) -> None:
    if isinstance(v, ConfigBase):
        _visit_configs(v, fn)
    elif isinstance(v, (list, tuple)):
        for x in v:
            _visit_value(x, fn)
    elif isinstance(v, dict):
        for x in v.values():
            _visit_value(x, fn)


def set_bias_recursively(cfg: ConfigBase, bias: bool = False) -> ConfigBase:
    """Sets every ``bias`` field in the tree."""

    def fn(c):
        if "bias" in c and isinstance(c.bias, bool):
            c.bias = bias

    _visit_configs(cfg, fn)
    return cfg


def set_norm_recursively(cfg: ConfigBase, norm_cfg: InstantiableConfig) -> ConfigBase:
    """Replaces every ``norm`` sub-config (keeping its ``input_dim``)."""

    def fn(c):
        if "norm" in c and isinstance(c.norm, ConfigBase):
            c.norm = norm_cfg.clone()
        for key in ("output_norm",):
            if key in c and isinstance(getattr(c, key), ConfigBase):
                setattr(c, key, norm_cfg.clone())

    _visit_configs(cfg, fn)
    return cfg


def set_dropout_rate_recursively(cfg: ConfigBase, dropout_rate: Optional[float]) -> ConfigBase:
    def fn(c):
        if "klass" in c and isinstance(c.klass, type) and issubclass(c.klass, Dropout):
            c.rate = dropout_rate
        if "dropout_rate" in c:
            c.dropout_rate = dropout_rate

    _visit_configs(cfg, fn)
    return cfg


def set_layer_norm_eps_recursively(cfg: ConfigBase, eps: float, set_only_if_none: bool = False) -> ConfigBase:
    def fn(c):
        if "klass" in c and isinstance(c.klass, type) and issubclass(c.klass, (LayerNormStateless, RMSNormStateless)):
            if not set_only_if_none or c.eps is None:
                c.eps = eps

    _visit_configs(cfg, fn)
    return cfg


# ------------------------------------------------------------------------------------------
# Classification metric layers (reference: axlearn/common/layers.py:984-1110).
# ------------------------------------------------------------------------------------------


class BaseClassificationMetric(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        num_classes: Required[int] = REQUIRED

    def forward(self, logits: Tensor, *, labels: Tensor, soft_labels: Optional[Tensor] = None) -> Tensor:
        raise NotImplementedError(type(self))


class ClassificationMetric(BaseClassificationMetric):
    """Softmax cross-entropy over in-range labels; logs loss, perplexity and accuracy."""

    @config_class
    class Config(BaseClassificationMetric.Config):
        label_smoothing: float = 0.0

    def forward(self, logits: Tensor, *, labels: Tensor, soft_labels: Optional[Tensor] = None) -> Tensor:
        from axlearn_b200.common.loss import cross_entropy
        from axlearn_b200.common.metrics import WeightedSummary

        cfg = self._config
        live = (labels >= 0) & (labels < cfg.num_classes)
        n = live.sum()
        loss, aux = cross_entropy(logits, labels, live_targets=live, label_smoothing=cfg.label_smoothing,
                                  soft_target_labels=soft_labels)
        accuracy = ((logits.argmax(dim=-1) == labels) & live).sum() / n.clamp_min(1)
        self.add_summary("loss", WeightedSummary(loss.detach(), n))
        self.add_summary("z_loss", WeightedSummary(aux["z_loss"].detach(), n))
        self.add_summary("cross_entropy_loss", WeightedSummary(aux["cross_entropy_loss"].detach(), n))
        self.add_summary("perplexity", WeightedSummary(torch.exp(loss.detach()), n))
        self.add_summary("accuracy", WeightedSummary(accuracy, n))
        return loss


class BinaryClassificationMetric(BaseClassificationMetric):
    """Sigmoid cross-entropy on 0/1 labels (other values are padding); logs precision, recall,
    F-score, loss and accuracy."""

    @config_class
    class Config(BaseClassificationMetric.Config):
        num_classes: int = 2
        prediction_threshold: float = 0.5

    def forward(self, logits: Tensor, *, labels: Tensor, soft_labels: Optional[Tensor] = None) -> Tensor:
        from axlearn_b200.common.metrics import WeightedSummary

        cfg = self._config
        if soft_labels is not None:
            raise ValueError("soft_labels must be None for binary classification")
        if cfg.num_classes != 2:
            raise ValueError(f"binary classification has two classes, got {cfg.num_classes}")
        live = (labels >= 0) & (labels < 2)
        n = live.sum()
        per = F.binary_cross_entropy_with_logits(logits.float(), labels.clamp(0, 1).float(), reduction="none")
        loss = (per * live).sum() / n.clamp_min(1)
        preds = (torch.sigmoid(logits.float()) > cfg.prediction_threshold) & live
        truth = (labels == 1) & live
        tp = (preds & truth).sum().float()
        precision = tp / preds.sum().clamp_min(1)
        recall = tp / truth.sum().clamp_min(1)
        f_score = 2 * precision * recall / (precision + recall).clamp_min(1e-12)
        accuracy = ((preds == truth) & live).sum() / n.clamp_min(1)
        self.add_summary("precision", precision)
        self.add_summary("recall", recall)
        self.add_summary("f_score", WeightedSummary(f_score, n))
        self.add_summary("loss", WeightedSummary(loss.detach(), n))
        self.add_summary("accuracy", WeightedSummary(accuracy, n))
        return loss
