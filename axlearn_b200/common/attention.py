"""Attention and transformer layers.

Parity targets in the reference (axlearn/common/attention.py): ``ForwardMode`` (:157),
``MultiheadOutputLinear`` (:536), ``QKVLinear`` (:729), ``GroupedQKVLinear`` (:790),
``QLinear`` (:819), ``FusedQKVLinear`` (:864), ``FusedGroupedQKVLinear`` (:984), RoPE
(:1063-1091, 1301-1349), ``RoFormerQKVLinear`` (:1553), ``ScaleQuery``/``ScaleKey``
(:1452-1550), ``MultiheadAttention`` (:1704), ``GroupedQueryAttention`` (:2383),
``TransformerAttentionLayer`` (:2779), ``TransformerFeedForwardLayer`` (:3114),
``TransformerLayer`` (:3413), ``StackedTransformerLayer`` (:3989),
``RepeatedTransformerLayer`` (:4373), ``build_remat_spec`` (:4574),
``set_double_shard_weights_config`` (:3803-3850).

Child and parameter names are the reference's, so state-tree paths such as
``.../self_attention/attention/i_proj/i_proj/qkv_proj/weight`` are unchanged.

Tensor parallelism: projection weights carry ``model`` on the heads / hidden dim.  Input
projections are column-parallel (local heads), ``o_proj`` and ``linear2`` are row-parallel
(partial sums reduced over ``model``).  Storage axes (``fsdp`` & co.) are gathered right
before use unless a prefetcher already did.
"""

from __future__ import annotations

import enum
import math
from typing import Any, Callable, NamedTuple, Optional, Sequence, Union

import torch

from axlearn_b200 import ops
from axlearn_b200.common import attention_bias as ab
from axlearn_b200.common import remat
from axlearn_b200.common.attention_bias import (
    NEG_INF,
    BaseAttentionBias,
    CausalAttentionBias,
    MaskFnAttentionBias,
    SegmentIdAttentionBias,
    SlidingWindowAttentionBias,
    TensorAttentionBias,
    ZeroAttentionBias,
    as_attention_bias,
)
from axlearn_b200.common.base_layer import (
    BaseLayer,
    FactorizationSpec,
    ParameterSpec,
    RematSpec,
    nothing_saveable,
)
from axlearn_b200.common.config import (
    REQUIRED,
    ConfigBase,
    InstantiableConfig,
    Required,
    config_class,
    config_for_function,
)
from axlearn_b200.common.kv_cache.base_kv_cache import BaseKVCache, KVState
from axlearn_b200.common.kv_cache.kv_cache import KVCache
from axlearn_b200.common.kv_cache.paged_kv_cache import materialize
from axlearn_b200.common.layers import (
    DenseGeneralBaseLayer,
    Dropout,
    LayerNorm,
    Linear,
    StochasticDepth,
    get_activation_fn,
)
from axlearn_b200.common.module import Module, nowrap
from axlearn_b200.common.param_init import FanAxes
from axlearn_b200.common.repeat import Repeat
from axlearn_b200.common.utils import Nested, VDict, tree_map
from axlearn_b200.parallel import collectives as coll

Tensor = torch.Tensor


class ForwardMode(enum.Enum):
    """FORWARD: plain call.  INIT_STATES: prefill that also builds the cache.
    EXTEND_STEP: consume and update the cache with new tokens."""

    FORWARD = 0
    INIT_STATES = 1
    EXTEND_STEP = 2


# ------------------------------------------------------------------------------------------
# Projections.
# ------------------------------------------------------------------------------------------


class MultiheadInputLinear(DenseGeneralBaseLayer):
    """``[B, T, D] -> [B, T, N, H]`` with weight ``[D, N, H]``."""

    @config_class
    class Config(DenseGeneralBaseLayer.Config):
        model_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        per_head_dim: Required[int] = REQUIRED
        bias: bool = True

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.param_partition_spec = (None, "model", None)
        return cfg

    def _create_layer_parameter_specs(self):
        cfg = self._config
        spec = cfg.param_partition_spec
        params = {
            "weight": ParameterSpec(
                shape=(cfg.model_dim, cfg.num_heads, cfg.per_head_dim),
                mesh_axes=spec,
                factorization=FactorizationSpec(axes=("row", None, "col")),
                fan_axes=FanAxes(in_axis=0, out_axis=(1, 2)),
            )
        }
        if cfg.bias:
            params["bias"] = ParameterSpec(
                shape=(cfg.num_heads, cfg.per_head_dim), mesh_axes=tuple(spec[1:]) if spec else None
            )
        return params

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        spec = cfg.param_partition_spec
        full = (cfg.model_dim, cfg.num_heads, cfg.per_head_dim)
        cshape = coll.compute_shape(full, spec)
        w = coll.unshard_param(self.parameters["weight"], spec, compute_shape=cshape)
        if coll.has_axis(spec[1] if spec else None, "model"):
            x = coll.tp_enter(x, "model")
        y = self._matmul(x, w.reshape(cshape[0], -1).to(x.dtype))
        y = y.reshape(x.shape[:-1] + (cshape[1], cshape[2]))
        if cfg.bias:
            b = coll.unshard_param(self.parameters["bias"], tuple(spec[1:]) if spec else None, compute_shape=cshape[1:])
            y = y + b.to(y.dtype)
        return y


class MultiheadOutputLinear(DenseGeneralBaseLayer):
    """``[B, T, N, H] -> [B, T, D]`` with weight ``[D, N, H]``."""

    @config_class
    class Config(DenseGeneralBaseLayer.Config):
        model_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        per_head_dim: Required[int] = REQUIRED
        bias: bool = True

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.param_partition_spec = (None, "model", None)
        return cfg

    def _create_layer_parameter_specs(self):
        cfg = self._config
        params = {
            "weight": ParameterSpec(
                shape=(cfg.model_dim, cfg.num_heads, cfg.per_head_dim),
                mesh_axes=cfg.param_partition_spec,
                factorization=FactorizationSpec(axes=("row", None, "col")),
                fan_axes=FanAxes(in_axis=(1, 2), out_axis=0),
            )
        }
        if cfg.bias:
            params["bias"] = ParameterSpec(shape=(cfg.model_dim,), mesh_axes=(None,))
        return params

    def forward(self, x: Tensor) -> Tensor:
        cfg = self._config
        spec = cfg.param_partition_spec
        full = (cfg.model_dim, cfg.num_heads, cfg.per_head_dim)
        cshape = coll.compute_shape(full, spec)
        w = coll.unshard_param(self.parameters["weight"], spec, compute_shape=cshape)
        w2 = w.reshape(cshape[0], -1).to(x.dtype)  # [D, N*H]
        x2 = x.reshape(x.shape[:-2] + (-1,))
        row_parallel = coll.has_axis(spec[1] if spec else None, "model")
        y = coll.row_parallel_linear(x2, w2.t(), "model") if row_parallel and self._plain_matmul() else None
        if y is None:
            y = self._matmul(x2, w2.t())
            if row_parallel:
                y = coll.tp_exit(y, "model")
        if cfg.bias:
            y = y + self.parameters["bias"].to(y.dtype)
        return y


class BaseQKVLinear(BaseLayer):
    """Maps (query, key, value) inputs to per-head projections."""

    @config_class
    class Config(BaseLayer.Config):
        query_dim: Required[int] = REQUIRED
        key_dim: Required[int] = REQUIRED
        value_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        per_head_dim: Required[int] = REQUIRED
        cache_dtype: Optional[torch.dtype] = None

    class Output(NamedTuple):
        query: Tensor
        key: Tensor
        value: Tensor

    @classmethod
    def is_kv_sharing(cls, cfg) -> bool:
        return False

    @property
    @nowrap
    def num_kv_heads(self) -> int:
        return self._config.num_heads

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        raise NotImplementedError(type(self))


def _proj_cfg(cfg, *, model_dim, num_heads):
    return cfg.layer.clone(model_dim=model_dim, num_heads=num_heads, per_head_dim=cfg.per_head_dim)


class QKVLinear(BaseQKVLinear):
    """Three separate projections ``q_proj``, ``k_proj``, ``v_proj``."""

    @config_class
    class Config(BaseQKVLinear.Config):
        layer: MultiheadInputLinear.Config = MultiheadInputLinear.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        for name, dim, heads in (
            ("q", cfg.query_dim, cfg.num_heads),
            ("k", cfg.key_dim, self.num_kv_heads),
            ("v", cfg.value_dim, self.num_kv_heads),
        ):
            self._add_child(f"{name}_proj", _proj_cfg(cfg, model_dim=dim, num_heads=heads))

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        if kv_state is not None:
            raise ValueError("QKVLinear does not take kv_state")
        key = query if key is None else key
        value = query if value is None else value
        return self.Output(self.q_proj(query), self.k_proj(key), self.v_proj(value))


class GroupedQKVLinear(QKVLinear):
    """QKVLinear with fewer key/value heads than query heads."""

    @config_class
    class Config(QKVLinear.Config):
        num_kv_heads: Required[int] = REQUIRED

    @property
    @nowrap
    def num_kv_heads(self) -> int:
        return self._config.num_kv_heads


class QLinear(BaseQKVLinear):
    """Projects queries only; keys/values come from another layer's ``kv_state``."""

    @config_class
    class Config(BaseQKVLinear.Config):
        layer: MultiheadInputLinear.Config = MultiheadInputLinear.default_config()

    @classmethod
    def is_kv_sharing(cls, cfg) -> bool:
        return True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("q_proj", _proj_cfg(cfg, model_dim=cfg.query_dim, num_heads=cfg.num_heads))

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        if kv_state is None:
            raise ValueError("QLinear needs kv_state")
        return self.Output(self.q_proj(query), kv_state.k_proj, kv_state.v_proj)


class _FusedQKVProj(DenseGeneralBaseLayer):
    """Weight ``[3, D, N, H]``: the three projections initialised from three keys."""

    @config_class
    class Config(DenseGeneralBaseLayer.Config):
        model_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        per_head_dim: Required[int] = REQUIRED
        bias: bool = True

    def _create_layer_parameter_specs(self):
        cfg = self._config
        spec = cfg.param_partition_spec
        params = {
            "weight": ParameterSpec(
                shape=(3, cfg.model_dim, cfg.num_heads, cfg.per_head_dim),
                mesh_axes=spec,
                factorization=FactorizationSpec(axes=(None, "row", None, "col")),
                fan_axes=FanAxes(in_axis=1, out_axis=(2, 3), batch_axis=0),
            )
        }
        if cfg.bias:
            params["bias"] = ParameterSpec(
                shape=(3, cfg.num_heads, cfg.per_head_dim),
                mesh_axes=(None,) + tuple(spec[2:]) if spec else None,
            )
        return params

    def forward(self, x: Tensor) -> tuple[Tensor, Tensor, Tensor]:
        cfg = self._config
        spec = cfg.param_partition_spec
        full = (3, cfg.model_dim, cfg.num_heads, cfg.per_head_dim)
        cshape = coll.compute_shape(full, spec)
        w = coll.unshard_param(self.parameters["weight"], spec, compute_shape=cshape)
        if coll.has_axis(spec[2] if spec else None, "model"):
            x = coll.tp_enter(x, "model")
        x = ops.share_input_grad(x)      # the three projections sum their input gradients in place
        outs = []
        for p in range(3):
            y = self._matmul(x, w[p].reshape(cshape[1], -1).to(x.dtype))
            y = y.reshape(x.shape[:-1] + (cshape[2], cshape[3]))
            if cfg.bias:
                y = y + self.parameters["bias"][p].to(y.dtype)
            outs.append(y)
        return tuple(outs)


class FusedQKVLinear(BaseQKVLinear):
    """Self-attention projections held in one parameter ``qkv_proj/weight [3, D, N, H]``."""

    @config_class
    class Config(BaseQKVLinear.Config):
        layer: InstantiableConfig = _FusedQKVProj.default_config().set(
            param_partition_spec=(None, None, "model", None)
        )

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if not cfg.query_dim == cfg.key_dim == cfg.value_dim:
            raise ValueError("FusedQKVLinear needs query_dim == key_dim == value_dim")
        layer = cfg.layer
        if layer.klass is MultiheadInputLinear:
            spec = layer.param_partition_spec
            layer = _FusedQKVProj.default_config().set(
                bias=layer.bias,
                param_partition_spec=(None,) + tuple(spec) if spec else None,
                quantized_dot_general=layer.quantized_dot_general,
            )
        self._add_child(
            "qkv_proj",
            layer.clone(model_dim=cfg.query_dim, num_heads=cfg.num_heads, per_head_dim=cfg.per_head_dim),
        )

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        if kv_state is not None:
            raise ValueError("FusedQKVLinear does not take kv_state")
        if key is not None or value is not None:
            raise ValueError("FusedQKVLinear supports self-attention only")
        return self.Output(*self.qkv_proj(query))


class FusedGroupedQKVLinear(BaseQKVLinear):
    """GQA projections in one parameter ``qkv_proj/weight [D, N + 2*Nkv, H]`` split on the
    head axis."""

    @config_class
    class Config(BaseQKVLinear.Config):
        num_kv_heads: Required[int] = REQUIRED
        layer: MultiheadInputLinear.Config = MultiheadInputLinear.default_config()

    @property
    @nowrap
    def num_kv_heads(self) -> int:
        return self._config.num_kv_heads

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if not cfg.query_dim == cfg.key_dim == cfg.value_dim:
            raise ValueError("FusedGroupedQKVLinear needs equal query/key/value dims")
        if cfg.num_heads % cfg.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self._add_child(
            "qkv_proj",
            cfg.layer.clone(
                model_dim=cfg.query_dim,
                num_heads=cfg.num_heads + 2 * cfg.num_kv_heads,
                per_head_dim=cfg.per_head_dim,
            ),
        )

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        cfg = self._config
        if kv_state is not None or key is not None or value is not None:
            raise ValueError("FusedGroupedQKVLinear supports self-attention only")
        proj = self.qkv_proj(query)  # [B, T, (N+2Nkv)/tp, H]
        tp = coll.axis_size("model") if coll.has_axis(
            (cfg.layer.param_partition_spec or (None, None, None))[1], "model") else 1
        if tp > 1:
            raise NotImplementedError(
                "FusedGroupedQKVLinear under tensor parallelism: use GroupedQKVLinear "
                "(a contiguous head split does not align q/k/v boundaries)"
            )
        n, nkv = cfg.num_heads, cfg.num_kv_heads
        q, k, v = torch.split(proj, [n, nkv, nkv], dim=-2)
        return self.Output(q, k, v)


# ------------------------------------------------------------------------------------------
# RoPE.
# ------------------------------------------------------------------------------------------


class RoFormerSinusoidalPositionalEmbedding(BaseLayer):
    """``[sin(p * f) | cos(p * f)]`` with ``f_i = theta^(-2i/dim)``."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        theta: float = 10000.0

    @nowrap
    def default_query_positions(self, max_seq_len: int, device=None) -> Tensor:
        return torch.arange(max_seq_len, device=device)[None]

    def forward(self, *, positions: Optional[Tensor] = None, max_seq_len: Optional[int] = None) -> Tensor:
        cfg = self._config
        if positions is None:
            positions = self.default_query_positions(max_seq_len)
        sin, cos = ops.reference.rope_tables(positions, cfg.dim, cfg.theta)
        return torch.cat([sin, cos], dim=-1)


class YaRNSinusoidalPositionalEmbedding(RoFormerSinusoidalPositionalEmbedding):
    """RoPE with YaRN context extension (arXiv:2309.00071; reference: axlearn/common/
    attention.py:1168-1298).  Dimensions that rotate fast (many periods within the original
    context) keep their frequency, slow ones are interpolated by ``scaling_factor``, with a linear
    ramp between the ``beta_fast`` and ``beta_slow`` rotation counts; sin / cos are multiplied by
    ``(0.1 ln(scaling_factor) + 1) * attn_factor``."""

    @config_class
    class Config(RoFormerSinusoidalPositionalEmbedding.Config):
        original_max_seq_length: Required[int] = REQUIRED
        scaling_factor: float = 1.0
        beta_slow: float = 1.0
        beta_fast: float = 32.0
        extrapolation_factor: float = 1.0
        attn_factor: float = 1.0

    @nowrap
    def compute_rope_params(self) -> tuple[Tensor, float]:
        """``(inverse frequencies [dim / 2], magnitude scale)``."""
        cfg = self._config
        dim, theta = cfg.dim, cfg.theta

        def correction_dim(rotations: float) -> float:
            # The dimension whose wavelength fits `rotations` times into the original context.
            return dim * math.log(cfg.original_max_seq_length / (rotations * 2 * math.pi)) / (2 * math.log(theta))

        pos_freqs = theta ** (2 * torch.arange(dim // 2, dtype=torch.float32) / dim)
        extrapolation = 1.0 / pos_freqs
        interpolation = 1.0 / (cfg.scaling_factor * pos_freqs)
        low = max(0, math.floor(correction_dim(cfg.beta_fast)))
        high = min(dim - 1, math.ceil(correction_dim(cfg.beta_slow)))
        if low == high:
            high += 0.001
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        mask = (1 - ramp) * cfg.extrapolation_factor
        inv_freq = interpolation * (1 - mask) + extrapolation * mask
        mscale = (0.1 * math.log(max(1.0, cfg.scaling_factor)) + 1.0) * cfg.attn_factor
        return inv_freq, mscale

    def forward(self, *, positions: Optional[Tensor] = None, max_seq_len: Optional[int] = None) -> Tensor:
        if positions is None:
            if max_seq_len is None:
                raise ValueError("need positions or max_seq_len")
            positions = self.default_query_positions(max_seq_len)
        inv_freq, mscale = self.compute_rope_params()
        enc = positions.float()[..., None] * inv_freq.to(positions.device)
        return torch.cat([torch.sin(enc) * mscale, torch.cos(enc) * mscale], dim=-1)


def apply_rotary_position_embeddings(
    *, query: Tensor, key: Tensor, value: Tensor, sinusoidal_pos: Tensor, rotary_key: bool = True,
    rotary_value: bool = False,
) -> tuple[Tensor, Tensor, Tensor]:
    """Rotates interleaved pairs; ``sinusoidal_pos``: ``[B, T, 1, H]`` = ``[sin | cos]``."""
    sin, cos = sinusoidal_pos.chunk(2, dim=-1)
    sin2 = torch.repeat_interleave(sin, 2, dim=-1)
    cos2 = torch.repeat_interleave(cos, 2, dim=-1)

    def rot(x):
        xf = x.float()
        r = torch.stack([-xf[..., 1::2], xf[..., 0::2]], dim=-1).reshape(x.shape)
        return (xf * cos2 + r * sin2).to(x.dtype)

    return rot(query), (rot(key) if rotary_key else key), (rot(value) if rotary_value else value)


class RoFormerQKVLinear(BaseQKVLinear):
    """Wraps another QKV projection and rotates q (and k, optionally v) by position."""

    @config_class
    class Config(BaseQKVLinear.Config):
        rope_pos_emb_layer: RoFormerSinusoidalPositionalEmbedding.Config = (
            RoFormerSinusoidalPositionalEmbedding.default_config()
        )
        input_linear: BaseQKVLinear.Config = QKVLinear.default_config()
        rotary_key: bool = True
        rotary_value: Required[bool] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("rope_pos_emb_layer", cfg.rope_pos_emb_layer.clone(dim=cfg.per_head_dim))
        self._add_child(
            "i_proj",
            cfg.input_linear.clone(
                query_dim=cfg.query_dim,
                key_dim=cfg.key_dim,
                value_dim=cfg.value_dim,
                num_heads=cfg.num_heads,
                per_head_dim=cfg.per_head_dim,
            ),
        )

    @property
    @nowrap
    def num_kv_heads(self) -> int:
        return self.i_proj.num_kv_heads

    def forward(self, query, *, key=None, value=None, kv_state=None, query_positions=None):
        cfg = self._config
        q, k, v = self.i_proj(query, key=key, value=value, kv_state=kv_state)
        if query_positions is None:
            query_positions = torch.arange(q.shape[1], device=q.device)
        theta = cfg.rope_pos_emb_layer.theta
        pos = query_positions
        if type(self.rope_pos_emb_layer) is not RoFormerSinusoidalPositionalEmbedding:  # pylint: disable=unidiomatic-typecheck
            # A scaled variant (e.g. YaRN): rotate with the layer's own sin / cos table.
            pos2 = pos if pos.dim() == 2 else pos[None]
            table = self.rope_pos_emb_layer(positions=pos2)[:, :, None, :]          # [B or 1, T, 1, H]
            if kv_state is not None:
                q, _, _ = apply_rotary_position_embeddings(
                    query=q, key=q, value=q, sinusoidal_pos=table, rotary_key=False, rotary_value=False)
                return self.Output(q, k, v)
            q, k, v = apply_rotary_position_embeddings(
                query=q, key=k, value=v, sinusoidal_pos=table, rotary_key=cfg.rotary_key,
                rotary_value=cfg.rotary_value)
            return self.Output(q, k, v)
        if pos.dim() == 2 and pos.shape[0] == 1:
            pos = pos[0]
        if kv_state is not None:
            # Keys of a shared KV state were rotated by the layer that produced them.
            return self.Output(ops.rope(q, pos, theta), k, v)
        q = ops.rope(q, pos, theta)
        if cfg.rotary_key:
            k = ops.rope(k, pos, theta)
        if cfg.rotary_value:
            v = ops.rope(v, pos, theta)
        return self.Output(q, k, v)


# ------------------------------------------------------------------------------------------
# Query / key scaling.
# ------------------------------------------------------------------------------------------


class PerDimScale(BaseLayer):
    """Learnable per-dimension scale ``softplus(param) * 1.442695 / ...``."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED

    def _create_layer_parameter_specs(self):
        from axlearn_b200.common.param_init import constant_initializer

        return {"param": ParameterSpec(shape=(self._config.dim,), mesh_axes=(None,), initializer=constant_initializer(0.0))}

    def forward(self, x: Tensor) -> Tensor:
        r_softplus_0 = 1.442695041
        return x * (r_softplus_0 * torch.nn.functional.softplus(self.parameters["param"])).to(x.dtype)


class BaseScaleQK(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        per_head_dim: Required[int] = REQUIRED
        norm: Optional[InstantiableConfig] = None
        # Callable (per_head_dim -> float) config or None for the default.
        scale_factor: Optional[InstantiableConfig] = None
        per_dim_scale: Optional[PerDimScale.Config] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.norm is not None:
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.per_head_dim))
        if cfg.per_dim_scale is not None:
            self._add_child("per_dim_scale", cfg.per_dim_scale.clone(dim=cfg.per_head_dim))
        self._scale_fn = cfg.scale_factor.instantiate() if cfg.scale_factor is not None else None

    @staticmethod
    def default_scale_factor(per_head_dim: int) -> float:
        raise NotImplementedError

    @nowrap
    def scale_value(self) -> float:
        d = self._config.per_head_dim
        return float(self._scale_fn(d)) if self._scale_fn is not None else float(self.default_scale_factor(d))

    @nowrap
    def is_pure_scalar(self) -> bool:
        return "norm" not in self._children and "per_dim_scale" not in self._children

    def apply_norm(self, x: Tensor) -> Tensor:
        if "norm" in self._children:
            x = self.norm(x)
        return x

    def apply_per_dim_scale(self, x: Tensor) -> Tensor:
        if "per_dim_scale" in self._children:
            x = self.per_dim_scale(x)
        return x

    def apply_scale_factor(self, x: Tensor) -> Tensor:
        s = self.scale_value()
        return x if s == 1.0 else x * s

    def forward(self, x: Tensor) -> Tensor:
        return self.apply_scale_factor(self.apply_per_dim_scale(self.apply_norm(x)))


class ScaleQuery(BaseScaleQK):
    """Default query scale ``per_head_dim ** -0.5``."""

    @staticmethod
    def default_scale_factor(per_head_dim: int) -> float:
        return per_head_dim**-0.5


class ScaleKey(BaseScaleQK):
    """Default key scale 1."""

    @staticmethod
    def default_scale_factor(per_head_dim: int) -> float:
        return 1.0


def constant_scale_fn(value: float) -> Callable[[int], float]:
    return lambda per_head_dim: value


def pow_scale_fn(exp: float) -> Callable[[int], float]:
    return lambda per_head_dim: per_head_dim**exp


# ------------------------------------------------------------------------------------------
# Multi-head attention.
# ------------------------------------------------------------------------------------------


def compute_padding_biases(paddings: Tensor) -> Tensor:
    """``[B, S]`` (1 = padding) -> additive ``[B, 1, 1, S]``."""
    return (paddings.float() * NEG_INF)[:, None, None, :]


class MultiheadAttention(BaseLayer):
    """Multi-head attention with optional KV cache (prefill / extend_step)."""

    @config_class
    class Config(BaseLayer.Config):
        query_dim: Required[int] = REQUIRED
        key_dim: Required[int] = REQUIRED
        value_dim: Required[int] = REQUIRED
        output_dim: Optional[int] = None
        hidden_dim: Optional[int] = None
        num_heads: Required[int] = REQUIRED
        input_linear: BaseQKVLinear.Config = QKVLinear.default_config()
        output_linear: MultiheadOutputLinear.Config = MultiheadOutputLinear.default_config()
        dropout: Dropout.Config = Dropout.default_config()
        query_scale: BaseScaleQK.Config = ScaleQuery.default_config()
        key_scale: Optional[BaseScaleQK.Config] = ScaleKey.default_config()
        atten_logit_cap: Optional[float] = None
        # Config of a MaskFnAttentionBias (e.g. config_for_class(CausalAttentionBias)).
        mask: Optional[InstantiableConfig] = None
        causal: Optional[bool] = None
        kv_cache: BaseKVCache.Config = KVCache.default_config()
        scale_kv_before_cache_update: Optional[bool] = None
        logit_sink: Optional[bool] = None
        # What to do with a ``seq`` mesh axis in self-attention: "ulysses" re-partitions q/k/v from
        # sequence-sharded to head-sharded with all-to-alls (reference: axlearn/common/
        # flash_attention/layer.py:165-216); "allgather_kv" keeps the queries sequence-sharded and
        # gathers K/V over the axis (context parallelism, reference: axlearn/common/
        # flash_attention/tpu_attention.py:1096-1283) -- the choice when there are fewer KV heads
        # than ranks or the head count does not divide.
        seq_parallel_mode: str = "ulysses"
        q_partition_spec: Optional[Sequence[Any]] = None
        k_partition_spec: Optional[Sequence[Any]] = None
        v_partition_spec: Optional[Sequence[Any]] = None
        o_partition_spec: Optional[Sequence[Any]] = None

    class Output(NamedTuple):
        data: Tensor
        probs: Optional[Tensor] = None
        kv_state: Optional[KVState] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.causal is not None and cfg.mask is not None:
            raise NotImplementedError("Cannot specify `causal` when using `mask`.")
        self._add_child(
            "i_proj",
            cfg.input_linear.clone(
                query_dim=cfg.query_dim,
                key_dim=cfg.key_dim,
                value_dim=cfg.value_dim,
                num_heads=cfg.num_heads,
                per_head_dim=self.per_head_dim(),
            ),
        )
        self._add_child(
            "o_proj",
            cfg.output_linear.clone(
                model_dim=self.output_dim(), num_heads=cfg.num_heads, per_head_dim=self.per_head_dim()
            ),
        )
        self._add_child("dropout", cfg.dropout)
        self._add_child("scale_query", cfg.query_scale.clone(per_head_dim=self.per_head_dim()))
        if cfg.key_scale is not None:
            self._add_child("scale_key", cfg.key_scale.clone(per_head_dim=self.per_head_dim()))
        self._add_child("kv_cache", cfg.kv_cache)

    @nowrap
    def hidden_dim(self) -> int:
        return self._config.hidden_dim or self._config.query_dim

    @nowrap
    def per_head_dim(self) -> int:
        cfg = self._config
        if self.hidden_dim() % cfg.num_heads:
            raise ValueError(f"num_heads {cfg.num_heads} must divide hidden_dim {self.hidden_dim()}")
        return self.hidden_dim() // cfg.num_heads

    @nowrap
    def output_dim(self) -> int:
        return self._config.output_dim or self._config.query_dim

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if cfg.logit_sink:
            from axlearn_b200.common.param_init import constant_initializer

            return {"sink": ParameterSpec(shape=(cfg.num_heads,), mesh_axes=("model",), initializer=constant_initializer(0.0))}
        return {}

    # -------------------------------------------------------------------------- mask helpers
    def _mask_kind(self) -> tuple[bool, Optional[int], Optional[Callable]]:
        """(is_causal, sliding_window, generic_mask_fn) described by cfg.causal / cfg.mask."""
        cfg = self._config
        if cfg.causal:
            return True, None, None
        if cfg.mask is None:
            return False, None, None
        klass = getattr(cfg.mask, "klass", None)
        if klass is CausalAttentionBias:
            return True, None, None
        if klass is SlidingWindowAttentionBias:
            return True, cfg.mask.sliding_window_size, None
        bias = cfg.mask.clone(shape=(1, 1)).instantiate()
        return False, None, bias.mask

    def _build_mask_bias(self, *, t: int, s: int, q_pos: Optional[Tensor], k_pos: Optional[Tensor]) -> Optional[BaseAttentionBias]:
        causal, window, fn = self._mask_kind()
        if window is not None:
            fn = ab.sliding_window_causal_mask(window)
        elif causal:
            fn = ab.causal_mask
        if fn is None:
            return None
        return MaskFnAttentionBias(mask=fn, shape=(t, s), target_positions=q_pos, source_positions=k_pos)

    # -------------------------------------------------------------------------- core
    def _forward_for_mode(
        self,
        *,
        mode: ForwardMode,
        query: Tensor,
        key: Optional[Tensor] = None,
        value: Optional[Tensor] = None,
        kv_state: Optional[KVState] = None,
        attention_logit_biases: Union[None, Tensor, BaseAttentionBias] = None,
        segment_ids: Optional[Tensor] = None,
        query_positions: Optional[Tensor] = None,
        cached_states: Optional[Nested] = None,
        return_aux: Optional[set] = None,
        page_pool: Optional[dict] = None,
    ) -> tuple[Optional[Nested], Optional["MultiheadAttention.Output"]]:
        cfg = self._config
        if (key is None) != (value is None):
            raise ValueError("key and value must be both None or both set")
        kv_sharing = cfg.input_linear.klass.is_kv_sharing(cfg.input_linear)
        if kv_sharing and kv_state is None:
            raise ValueError("kv_state must be provided for KV sharing layers")
        if kv_state is not None and key is not None:
            raise ValueError("kv_state should not be specified together with key/value")
        kv_kwargs: dict[str, Any] = {}
        if kv_state is not None:
            kv_kwargs["kv_state"] = kv_state
        elif key is not None:
            kv_kwargs.update(key=key, value=value)
        is_self_attention = key is None and kv_state is None
        b, t = query.shape[:2]
        if coll.tp_sequence_parallel_dim() is not None and is_self_attention:
            # Sequence-sharded tensor-parallel region: `query` is this rank's slice; the projections
            # all-gather it, so everything below sees the whole sequence.
            t = t * coll.axis_size("model")
        dev = query.device
        default_positions = query_positions is None
        # Ulysses sequence parallelism: activations hold this rank's contiguous slice of the
        # sequence; attention itself runs on whole sequences with a slice of the heads.
        sp = _seq_parallel_size() if (mode == ForwardMode.FORWARD and is_self_attention) else 1
        if query_positions is None:
            query_positions = torch.arange(t, device=dev)[None]
            if sp > 1:
                query_positions = query_positions + coll.axis_index("seq") * t
        elif query_positions.dim() == 1:
            query_positions = query_positions[None]
        key_positions = (
            torch.arange(key.shape[1], device=dev)[None] if key is not None else query_positions
        )
        if mode in (ForwardMode.INIT_STATES, ForwardMode.EXTEND_STEP):
            time_step = cached_states["time_step"]
            query_positions = query_positions + time_step[:, None]
            key_positions = key_positions + time_step[:, None] if key is None else key_positions
        with remat.tagged(self, ("q_proj", "k_proj", "v_proj")):
            q_proj, k_proj, v_proj = self.i_proj(query, query_positions=query_positions, **kv_kwargs)
        q_proj = self._remat_name(q_proj, "q_proj")
        k_proj = self._remat_name(k_proj, "k_proj")
        v_proj = self._remat_name(v_proj, "v_proj")

        # Query/key scaling. A pure scalar scale is folded into the softmax scale of the
        # fused kernel instead of a separate pass over q.
        softmax_scale = 1.0
        if self.scale_query.is_pure_scalar():
            softmax_scale *= self.scale_query.scale_value()
        else:
            q_proj = self.scale_query(q_proj)
        if "scale_key" in self._children and not kv_sharing:
            if self.scale_key.is_pure_scalar():
                softmax_scale *= self.scale_key.scale_value()
            else:
                k_proj = self.scale_key(k_proj)

        cp_kv = None  # context parallelism: (gathered K, gathered V, key segment ids, first query position)
        if sp > 1 and cfg.seq_parallel_mode == "allgather_kv":
            if not default_positions:
                raise NotImplementedError("sequence parallelism needs default (contiguous) positions")
            rank = coll.axis_index("seq")
            k_all = coll.all_gather(k_proj.contiguous(), "seq", dim=1)   # backward: reduce-scatter of dK
            v_all = coll.all_gather(v_proj.contiguous(), "seq", dim=1)
            kv_seg = None
            if segment_ids is not None:
                kv_seg = coll.all_gather_raw(segment_ids.contiguous(), coll.current_group("seq"), sp, 1)
            cp_kv = (k_all, v_all, kv_seg, rank * t)
            sp = 1  # everything after the attention stays sequence-sharded
        elif sp > 1:
            if cfg.seq_parallel_mode != "ulysses":
                raise ValueError(f"unknown seq_parallel_mode {cfg.seq_parallel_mode!r}")
            if not default_positions:
                raise NotImplementedError("sequence parallelism needs default (contiguous) positions")
            q_proj, k_proj, v_proj = (_seq_to_heads(x, sp) for x in (q_proj, k_proj, v_proj))
            t = t * sp
            query_positions = key_positions = torch.arange(t, device=dev)[None]
            if segment_ids is not None:
                segment_ids = coll.all_gather_raw(
                    segment_ids.contiguous(), coll.current_group("seq"), sp, 1)
        new_cached_states = None
        live_kv: Optional[KVState] = None
        if mode == ForwardMode.FORWARD:
            if kv_state is not None:
                key_positions = kv_state.key_positions
            live_kv = KVState(k_proj=k_proj, v_proj=v_proj, key_positions=key_positions)
        else:
            live_step_len = None
            if mode == ForwardMode.INIT_STATES and segment_ids is not None:
                live_step_len = (segment_ids != 0).sum(dim=-1)
            if kv_sharing:
                live_kv = kv_state
                new_cached_states = {"time_step": time_step + (live_step_len if live_step_len is not None else t)}
            else:
                kv_cached, live_kv = self.kv_cache.extend_step(
                    cached_states["kv_cache"],
                    k_proj=k_proj,
                    v_proj=v_proj,
                    key_positions=key_positions,
                    live_step_len=live_step_len,
                    page_pool=page_pool,
                )
                new_cached_states = {
                    "kv_cache": kv_cached,
                    "time_step": time_step + (live_step_len if live_step_len is not None else t),
                }

        # Assemble biases.
        user_bias = as_attention_bias(attention_logit_biases)
        dense_kv = materialize(live_kv)
        s = dense_kv.k_proj.shape[1]
        causal, window, generic_fn = self._mask_kind()
        # The fused kernel assumes positions 0..T-1 on both sides, which holds for plain
        # self-attention called without explicit positions.
        plain_positions = mode == ForwardMode.FORWARD and is_self_attention and default_positions
        want_probs = return_aux is not None and "probs" in return_aux
        # Causal, sliding-window, segment-id and logit-cap masking all happen inside the attention
        # kernel; an arbitrary bias, a logit sink, dropout or a request for the probabilities need
        # the materialised path.
        fast = (
            plain_positions
            and not user_bias.has_value()
            and generic_fn is None
            and (window is None or causal)
            and not cfg.logit_sink
            and not want_probs
            and not (self.is_training and cfg.dropout.rate)
        )
        if cp_kv is not None:
            if not fast:
                raise NotImplementedError("allgather_kv context parallelism supports the kernel masks only "
                                          "(causal, sliding window, segment ids, logit cap)")
            k_all, v_all, kv_seg, q_start = cp_kv
            if causal:
                # Queries are positions [q_start, q_start + t): keys beyond the last query are never
                # visible, and dropping them makes the queries the LAST t positions of the keys,
                # which is the offset convention of the attention op.
                k_all, v_all = k_all[:, : q_start + t], v_all[:, : q_start + t]
                kv_seg = None if kv_seg is None else kv_seg[:, : q_start + t]
            with remat.tagged(self, "context"):
                context = ops.attention(
                    q_proj, k_all, v_all, causal=causal, softmax_scale=softmax_scale,
                    segment_ids=segment_ids, kv_segment_ids=kv_seg, sliding_window=window,
                    logit_cap=cfg.atten_logit_cap, q_offset=(q_start if causal else None),
                )
            probs = None
        elif fast:
            with remat.tagged(self, "context"):
                context = ops.attention(
                    q_proj, dense_kv.k_proj, dense_kv.v_proj, causal=causal,
                    softmax_scale=softmax_scale, segment_ids=segment_ids,
                    sliding_window=window, logit_cap=cfg.atten_logit_cap,
                )
            probs = None
        else:
            biases: list[BaseAttentionBias] = [user_bias]
            mask_bias = self._build_mask_bias(
                t=t, s=s, q_pos=query_positions, k_pos=dense_kv.key_positions
            )
            if mask_bias is not None:
                biases.append(mask_bias)
            if segment_ids is not None and mode == ForwardMode.FORWARD:
                biases.append(SegmentIdAttentionBias(segment_ids=segment_ids))
            if mode != ForwardMode.FORWARD or kv_state is not None:
                # Slots holding no valid key (negative position) must never be attended.
                kp = dense_kv.key_positions
                if (kp < 0).any():
                    biases.append(TensorAttentionBias.from_tensor(
                        torch.where(kp >= 0, 0.0, NEG_INF)[:, None, None, :].expand(-1, 1, 1, -1)))
            bias_val = ab.CompositeAttentionBias(biases).value()
            context, probs = self._compute_attention(
                q_proj=q_proj, k_proj=dense_kv.k_proj, v_proj=dense_kv.v_proj,
                bias=bias_val, softmax_scale=softmax_scale, want_probs=want_probs,
            )
        if sp > 1:
            context = coll.all_to_all(context, "seq", split_dim=1, concat_dim=2)
        context = self._remat_name(context, "context")
        with remat.tagged(self, "o_proj"):
            o = self.o_proj(context)
        o = self._remat_name(o, "o_proj")
        out_kv = None
        if return_aux is not None and "kv_state" in return_aux:
            out_kv = live_kv if mode != ForwardMode.FORWARD else KVState(k_proj, v_proj, key_positions)
        return new_cached_states, self.Output(data=o, probs=probs, kv_state=out_kv)

    def _compute_attention(self, *, q_proj, k_proj, v_proj, bias, softmax_scale, want_probs):
        """Generic (bias-tensor) attention path."""
        cfg = self._config
        dropout_mask = None
        if self.is_training and cfg.dropout.rate:
            from axlearn_b200.common import prng

            b, t, n, _ = q_proj.shape
            keep = prng.bernoulli(self.prng_key, 1 - cfg.dropout.rate, (b, n, t, k_proj.shape[1]), device=q_proj.device)
            dropout_mask = keep.float() / (1 - cfg.dropout.rate)
        if cfg.logit_sink:
            return self._attention_with_sink(q_proj, k_proj, v_proj, bias, softmax_scale, dropout_mask)
        out = ops.reference.attention(
            q_proj, k_proj.to(q_proj.dtype), v_proj.to(q_proj.dtype), bias=bias, softmax_scale=softmax_scale,
            logit_cap=cfg.atten_logit_cap, dropout_mask=dropout_mask, return_probs=want_probs,
        )
        if want_probs:
            return out
        return out, None

    def _attention_with_sink(self, q, k, v, bias, scale, dropout_mask):
        b, t, n, h = q.shape
        nkv = k.shape[2]
        g = n // nkv
        logits = torch.einsum("btkgh,bskh->bkgts", q.float().reshape(b, t, nkv, g, h), k.float()).reshape(b, n, t, -1) * scale
        if self._config.atten_logit_cap:
            c = self._config.atten_logit_cap
            logits = c * torch.tanh(logits / c)
        if bias is not None:
            logits = logits + bias.float()
        sink = self.parameters["sink"].float()[None, :, None, None].expand(b, -1, t, 1)
        probs = torch.softmax(torch.cat([logits, sink], dim=-1), dim=-1)[..., :-1]
        if dropout_mask is not None:
            probs = probs * dropout_mask
        ctx = torch.einsum("bkgts,bskh->btkgh", probs.reshape(b, nkv, g, t, -1), v.float()).reshape(b, t, n, h)
        return ctx.to(q.dtype), probs

    # -------------------------------------------------------------------------- public API
    def forward(
        self,
        query: Tensor,
        *,
        key: Optional[Tensor] = None,
        value: Optional[Tensor] = None,
        kv_state: Optional[KVState] = None,
        attention_logit_biases: Union[None, Tensor, BaseAttentionBias] = None,
        segment_ids: Optional[Tensor] = None,
        query_positions: Optional[Tensor] = None,
        return_aux: Optional[set] = None,
    ) -> "MultiheadAttention.Output":
        _, out = self._forward_for_mode(
            mode=ForwardMode.FORWARD, query=query, key=key, value=value, kv_state=kv_state,
            attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
            query_positions=query_positions, return_aux=return_aux,
        )
        return out

    def init_states(
        self,
        *,
        time_step: Optional[Tensor],
        query: Union[Tensor, Any],
        key: Optional[Tensor] = None,
        value: Optional[Tensor] = None,
        kv_state: Optional[KVState] = None,
        attention_logit_biases: Union[None, Tensor, BaseAttentionBias] = None,
        segment_ids: Optional[Tensor] = None,
        return_aux: Optional[set] = None,
        page_pool: Optional[dict] = None,
        max_len: Optional[int] = None,
    ):
        """Builds the cache.  With ``time_step=None`` only allocates (``query`` may be a
        TensorSpec-like with ``shape``/``dtype``); otherwise also prefills from ``query``
        where ``time_step[b]`` is the number of valid prompt tokens."""
        cfg = self._config
        b, t = query.shape[:2]
        dtype = query.dtype or torch.float32
        dev = getattr(query, "device", None)
        kv_len = max_len or t
        init: dict[str, Any] = {"time_step": torch.zeros(b, dtype=torch.int32, device=dev)}
        if not cfg.input_linear.klass.is_kv_sharing(cfg.input_linear):
            init["kv_cache"] = self.kv_cache.init_states(
                BaseKVCache.Shape(b, kv_len, self.i_proj.num_kv_heads // self._tp_heads_div(), self.per_head_dim()),
                dtype=dtype, device=dev,
            )
        if time_step is None:
            return init, None
        if segment_ids is None:
            segment_ids = (torch.arange(t, device=dev)[None] < time_step[:, None]).to(torch.int32)
        return self._forward_for_mode(
            mode=ForwardMode.INIT_STATES, query=query, key=key, value=value, kv_state=kv_state,
            attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
            cached_states=init, return_aux=return_aux, page_pool=page_pool,
        )

    def _tp_heads_div(self) -> int:
        return 1

    def prefill_states(self, *, time_step: Tensor, query: Tensor, **kwargs):
        return self.init_states(time_step=time_step, query=query, **kwargs)

    def extend_step(
        self,
        cached_states: Nested,
        query: Tensor,
        *,
        key: Optional[Tensor] = None,
        value: Optional[Tensor] = None,
        kv_state: Optional[KVState] = None,
        attention_logit_biases: Union[None, Tensor, BaseAttentionBias] = None,
        return_aux: Optional[set] = None,
        page_pool: Optional[dict] = None,
    ):
        return self._forward_for_mode(
            mode=ForwardMode.EXTEND_STEP, query=query, key=key, value=value, kv_state=kv_state,
            attention_logit_biases=attention_logit_biases, cached_states=cached_states,
            return_aux=return_aux, page_pool=page_pool,
        )


def _seq_parallel_size() -> int:
    from axlearn_b200.parallel.mesh import current_mesh

    mesh = current_mesh()
    return mesh.shape.get("seq", 1) if mesh is not None else 1


def _seq_to_heads(x: Tensor, sp: int) -> Tensor:
    """``[B, T/sp, N, H] -> [B, T, N/sp, H]`` by an all-to-all over the ``seq`` axis; KV heads are
    repeated first when there are fewer of them than ranks (reference:
    axlearn/common/flash_attention/layer.py:204-216)."""
    n = x.shape[2]
    if n % sp:
        if sp % n:
            raise ValueError(f"{n} heads cannot be split over a seq axis of {sp}")
        x = x.repeat_interleave(sp // n, dim=2)
    return coll.all_to_all(x.contiguous(), "seq", split_dim=2, concat_dim=1)


class GroupedQueryAttention(MultiheadAttention):
    """Attention whose input projection yields fewer KV heads than query heads; the grouped
    contraction never repeats K/V in memory."""

    @nowrap
    def num_kv_heads(self) -> int:
        return self.i_proj.num_kv_heads


class SigmoidAttention(MultiheadAttention):
    """Attention with element-wise sigmoid instead of softmax (bias ``-log(seq_len)``)."""

    @config_class
    class Config(MultiheadAttention.Config):
        seq_len: Required[int] = REQUIRED
        subtract_seq_len_bias: bool = True

    def _compute_attention(self, *, q_proj, k_proj, v_proj, bias, softmax_scale, want_probs):
        cfg = self._config
        b, t, n, h = q_proj.shape
        nkv = k_proj.shape[2]
        g = n // nkv
        logits = torch.einsum("btkgh,bskh->bkgts", q_proj.float().reshape(b, t, nkv, g, h), k_proj.float()).reshape(b, n, t, -1) * softmax_scale
        if bias is not None:
            logits = logits + bias.float()
        if cfg.subtract_seq_len_bias:
            logits = logits - math.log(cfg.seq_len)
        probs = torch.sigmoid(logits)
        ctx = torch.einsum("bkgts,bskh->btkgh", probs.reshape(b, nkv, g, t, -1), v_proj.float()).reshape(b, t, n, h)
        return ctx.to(q_proj.dtype), (probs if want_probs else None)


# ------------------------------------------------------------------------------------------
# Transformer blocks.
# ------------------------------------------------------------------------------------------


class TransformerAttentionLayer(BaseLayer):
    """Norm + attention + residual, in one of the structures prenorm / postnorm /
    hybridnorm."""

    @config_class
    class Config(BaseLayer.Config):
        target_dim: Required[int] = REQUIRED
        source_dim: Required[int] = REQUIRED
        norm: InstantiableConfig = LayerNorm.default_config()
        attention: InstantiableConfig = MultiheadAttention.default_config()
        dropout: InstantiableConfig = Dropout.default_config()
        stochastic_depth: InstantiableConfig = StochasticDepth.default_config()
        structure: str = "prenorm"

    class Output(NamedTuple):
        data: Tensor
        probs: Optional[Tensor] = None
        kv_state: Optional[KVState] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.structure in ("prenorm", "postnorm"):
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.target_dim))
        elif cfg.structure == "hybridnorm":
            self._add_child("prenorm", cfg.norm.clone(input_dim=cfg.target_dim))
            self._add_child("postnorm", cfg.norm.clone(input_dim=cfg.target_dim))
        else:
            raise NotImplementedError(cfg.structure)
        self._add_child(
            "attention",
            cfg.attention.clone(
                query_dim=cfg.target_dim, key_dim=cfg.source_dim, value_dim=cfg.source_dim,
                output_dim=cfg.target_dim,
            ),
        )
        self._add_child("dropout", cfg.dropout)
        self._add_child("stochastic_depth", cfg.stochastic_depth)

    def _forward_for_mode(self, *, mode, target, source=None, attention_logit_biases=None,
                          segment_ids=None, target_positions=None, cached_states=None,
                          return_aux=None, page_pool=None, max_len=None, defer_residual=False):
        cfg = self._config
        kv_kwargs: dict[str, Any] = {}
        if isinstance(source, KVState):
            kv_kwargs["kv_state"] = source
        elif source is not None:
            kv_kwargs.update(key=source, value=source)

        def attend(x):
            if mode == ForwardMode.FORWARD:
                return None, self.attention(
                    query=x, attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
                    query_positions=target_positions, return_aux=return_aux, **kv_kwargs)
            if mode == ForwardMode.INIT_STATES:
                return self.attention.init_states(
                    time_step=cached_states["attention"], query=x,
                    attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
                    return_aux=return_aux, page_pool=page_pool, max_len=max_len, **kv_kwargs)
            return self.attention.extend_step(
                cached_states["attention"], x, attention_logit_biases=attention_logit_biases,
                return_aux=return_aux, page_pool=page_pool, **kv_kwargs)

        if mode == ForwardMode.INIT_STATES and cached_states["attention"] is None:
            states, _ = self.attention.init_states(time_step=None, query=target, page_pool=page_pool, **kv_kwargs)
            return {"attention": states}, None
        if cfg.structure == "prenorm":
            if mode == ForwardMode.FORWARD and hasattr(self.norm, "forward_keep_input"):
                normed, skip = self.norm.forward_keep_input(target)
            else:
                normed, skip = self.norm(target), target
            states, out = attend(normed)
            branch = self.stochastic_depth(self.dropout(out.data))
            # With `defer_residual` the caller adds the branch (fused into its next norm).
            data = (skip, branch) if defer_residual else skip + branch
        elif cfg.structure == "postnorm":
            states, out = attend(target)
            data = self.norm(target + self.stochastic_depth(self.dropout(out.data)))
        else:
            skip = target
            states, out = attend(self.prenorm(target))
            data = skip + self.stochastic_depth(self.dropout(self.postnorm(out.data)))
        return {"attention": states}, self.Output(data=data, probs=out.probs, kv_state=out.kv_state)

    def forward(self, *, target, source=None, attention_logit_biases=None, segment_ids=None,
                target_positions=None, return_aux=None, defer_residual: bool = False):
        """``defer_residual`` (pre-norm structure only): ``Output.data`` is the pair
        ``(skip, branch)`` instead of their sum, for a caller that fuses the addition into the
        next normalisation."""
        if defer_residual and self._config.structure != "prenorm":
            raise ValueError("defer_residual needs the prenorm structure")
        _, out = self._forward_for_mode(
            mode=ForwardMode.FORWARD, target=target, source=source,
            attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
            target_positions=target_positions, return_aux=return_aux, defer_residual=defer_residual)
        return out

    def init_states(self, *, time_step, target, source=None, attention_logit_biases=None,
                    segment_ids=None, return_aux=None, page_pool=None, max_len=None):
        if time_step is None:
            kv_kwargs = {"kv_state": source} if isinstance(source, KVState) else {}
            states, _ = self.attention.init_states(time_step=None, query=target, page_pool=page_pool, max_len=max_len, **kv_kwargs)
            return {"attention": states}, None
        return self._forward_for_mode(
            mode=ForwardMode.INIT_STATES, target=target, source=source,
            attention_logit_biases=attention_logit_biases, segment_ids=segment_ids,
            cached_states={"attention": time_step}, return_aux=return_aux, page_pool=page_pool,
            max_len=max_len)

    def extend_step(self, cached_states, target, *, source=None, attention_logit_biases=None,
                    return_aux=None, page_pool=None):
        return self._forward_for_mode(
            mode=ForwardMode.EXTEND_STEP, target=target, source=source,
            attention_logit_biases=attention_logit_biases, cached_states=cached_states,
            return_aux=return_aux, page_pool=page_pool)


def scaled_hidden_dim(scale: float = 4, *, round_up_to_multiples_of: Optional[int] = None):
    """Config of ``input_dim -> hidden_dim`` used by feed-forward layers; e.g.
    ``scaled_hidden_dim(8/3, round_up_to_multiples_of=256)`` gives 11008 for 4096."""

    def scale_fn(input_dim: int, *, scale: float, round_up_to_multiples_of: Optional[int]) -> int:
        hidden = input_dim * scale
        if round_up_to_multiples_of:
            hidden = math.ceil(hidden / round_up_to_multiples_of) * round_up_to_multiples_of
        return int(hidden)

    return config_for_function(scale_fn).set(scale=scale, round_up_to_multiples_of=round_up_to_multiples_of)


def _first_model_axis(linear) -> Any:
    """Output-dim entry of a linear's partition spec (tensor parallel layers route their input
    through a gradient all-reduce, which makes a new tensor per linear)."""
    spec = getattr(linear.config, "param_partition_spec", None)
    return spec[-1] if spec else None


class TransformerFeedForwardLayer(BaseLayer):
    """Norm + MLP + residual.  ``activation`` is a name, or a pair of names for a gated MLP
    (children ``linear1_0`` / ``linear1_1``): SwiGLU = ("nn.silu", "linear")."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        hidden_dim: Required[Union[int, InstantiableConfig]] = REQUIRED
        linear1: Linear.Config = Linear.default_config().set(param_partition_spec=(None, "model"))
        linear2: Linear.Config = Linear.default_config().set(param_partition_spec=("model", None))
        norm: InstantiableConfig = LayerNorm.default_config()
        activation: Union[str, tuple] = "nn.relu"
        dropout: InstantiableConfig = Dropout.default_config()
        stochastic_depth: InstantiableConfig = StochasticDepth.default_config()
        structure: str = "prenorm"
        residual_weight: float = 1.0
        add_dead_neuron_summary: Optional[bool] = None
        add_value_rms_norm_summary: Sequence[str] = ()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        hidden = cfg.hidden_dim
        if isinstance(hidden, InstantiableConfig):
            hidden = hidden.clone(input_dim=cfg.input_dim).instantiate()
        self._hidden_dim = int(hidden)
        if cfg.structure in ("prenorm", "postnorm"):
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.input_dim))
        elif cfg.structure == "hybridnorm":
            self._add_child("prenorm", cfg.norm.clone(input_dim=cfg.input_dim))
            self._add_child("postnorm", cfg.norm.clone(input_dim=cfg.input_dim))
        elif cfg.structure != "nonorm":
            raise NotImplementedError(cfg.structure)
        if isinstance(cfg.activation, (tuple, list)):
            if len(cfg.activation) != 2:
                raise ValueError("gated activation needs exactly two entries")
            for i in range(2):
                self._add_child(f"linear1_{i}", cfg.linear1.clone(input_dim=cfg.input_dim, output_dim=self._hidden_dim))
        else:
            self._add_child("linear1", cfg.linear1.clone(input_dim=cfg.input_dim, output_dim=self._hidden_dim))
        self._add_child("linear2", cfg.linear2.clone(input_dim=self._hidden_dim, output_dim=cfg.input_dim))
        if cfg.structure in ("prenorm", "hybridnorm", "nonorm"):
            self._add_child("dropout1", cfg.dropout)
            self._add_child("dropout2", cfg.dropout)
        else:
            self._add_child("dropout1", cfg.dropout)
            self._add_child("dropout2", cfg.dropout)
        self._add_child("stochastic_depth", cfg.stochastic_depth)

    @nowrap
    def hidden_dim(self) -> int:
        return self._hidden_dim

    def _mlp(self, x: Tensor) -> Tensor:
        cfg = self._config
        if isinstance(cfg.activation, (tuple, list)):
            if not coll.has_axis(_first_model_axis(self.linear1_0), "model"):
                x = ops.share_input_grad(x)  # both halves sum their input gradients in place
            with remat.tagged(self, "linear1_0"):
                a0 = self._remat_name(self.linear1_0(x), "linear1_0")
            with remat.tagged(self, "linear1_1"):
                a1 = self._remat_name(self.linear1_1(x), "linear1_1")
            if tuple(cfg.activation) == ("nn.silu", "linear"):
                h = ops.swiglu(a0, a1)
            elif tuple(cfg.activation) == ("linear", "nn.silu"):
                h = ops.swiglu(a1, a0)
            else:
                h = get_activation_fn(cfg.activation[0])(a0) * get_activation_fn(cfg.activation[1])(a1)
        else:
            with remat.tagged(self, "linear1_0"):
                h = get_activation_fn(cfg.activation)(self._remat_name(self.linear1(x), "linear1_0"))
        if cfg.add_dead_neuron_summary:
            self.add_summary("dead_neurons", (h.detach() <= 0).float().mean())
        h = self.dropout1(h)
        with remat.tagged(self, "linear2"):
            return self._remat_name(self.linear2(h), "linear2")

    ACCEPTS_PENDING_RESIDUAL = True

    def forward(self, inputs: Tensor, *, pending_residual: Optional[Tensor] = None) -> Tensor:
        """``pending_residual`` (pre-norm structure only): a branch output that still has to be
        added to ``inputs``; the addition is fused into this layer's normalisation."""
        cfg = self._config
        rw = cfg.residual_weight
        if pending_residual is not None and cfg.structure != "prenorm":
            inputs, pending_residual = inputs + pending_residual, None
        if cfg.structure == "prenorm":
            if pending_residual is not None and hasattr(self.norm, "forward_add"):
                inputs, normed = self.norm.forward_add(inputs, pending_residual)
            else:
                if pending_residual is not None:
                    inputs = inputs + pending_residual
                if hasattr(self.norm, "forward_keep_input"):
                    normed, inputs = self.norm.forward_keep_input(inputs)
                else:
                    normed = self.norm(inputs)
            x = self._mlp(normed)
            x = self.stochastic_depth(self.dropout2(x))
            return inputs + (x if rw == 1.0 else x * rw)
        if cfg.structure == "postnorm":
            x = self.stochastic_depth(self.dropout2(self._mlp(inputs)))
            return self.norm((x if rw == 1.0 else x * rw) + inputs)
        if cfg.structure == "hybridnorm":
            x = self.postnorm(self._mlp(self.prenorm(inputs)))
            x = self.stochastic_depth(self.dropout2(x))
            return inputs + (x if rw == 1.0 else x * rw)
        x = self.stochastic_depth(self.dropout2(self._mlp(inputs)))
        return inputs + (x if rw == 1.0 else x * rw)


class BaseTransformerLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED

    class Output(NamedTuple):
        data: Tensor
        self_attention_probs: Optional[Tensor] = None
        self_attention_kv_state: Optional[KVState] = None
        cross_attention_probs: Optional[Tensor] = None

    def forward(self, data, *, self_attention_logit_biases=None, cross_attention_data=None,
                cross_attention_logit_biases=None, target_segment_ids=None, target_positions=None,
                return_aux=None):
        raise NotImplementedError(type(self))


class TransformerLayer(BaseTransformerLayer):
    """self_attention -> [cross_attention] -> feed_forward."""

    @config_class
    class Config(BaseTransformerLayer.Config):
        self_attention: InstantiableConfig = TransformerAttentionLayer.default_config()
        cross_attention: Optional[InstantiableConfig] = None
        feed_forward: InstantiableConfig = TransformerFeedForwardLayer.default_config()
        # With a `model` mesh axis: the layer's input and output are 1 / tp slices of the
        # sequence (dim 1); norms and residual adds work on the slice, column-parallel linears
        # all-gather their input and row-parallel linears reduce-scatter their output.  Set by
        # the stack (``BaseStackedTransformerLayer.Config.tp_sequence_parallel``), which also
        # slices the stack's input and gathers its output.
        tp_sequence_parallel: bool = False

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("self_attention", cfg.self_attention.clone(target_dim=cfg.input_dim, source_dim=cfg.input_dim))
        self._add_child("feed_forward", cfg.feed_forward.clone(input_dim=cfg.input_dim))
        if cfg.cross_attention is not None:
            self._add_child("cross_attention", cfg.cross_attention.clone(target_dim=cfg.input_dim))

    def _forward_for_mode(self, *, mode, data, self_attention_kv_state=None,
                          self_attention_logit_biases=None, cross_attention_data=None,
                          cross_attention_logit_biases=None, target_segment_ids=None,
                          target_positions=None, cached_states=None, return_aux=None, page_pool=None,
                          max_len=None):
        data = self._remat_name(data, "input") if isinstance(data, Tensor) else data
        sa_kwargs = dict(target=data, source=self_attention_kv_state,
                         attention_logit_biases=self_attention_logit_biases, return_aux=return_aux)
        # Pre-norm blocks hand the attention branch to the feed-forward layer unsummed: its
        # normalisation adds it (one pass instead of an add and a norm).
        defer = (mode == ForwardMode.FORWARD and self.self_attention.config.structure == "prenorm"
                 and getattr(self.feed_forward, "ACCEPTS_PENDING_RESIDUAL", False)
                 and not (cross_attention_data is not None and "cross_attention" in self._children))
        if mode == ForwardMode.FORWARD:
            states, sa = None, self.self_attention(
                segment_ids=target_segment_ids, target_positions=target_positions, defer_residual=defer, **sa_kwargs)
        elif mode == ForwardMode.INIT_STATES:
            states, sa = self.self_attention.init_states(
                time_step=cached_states["self_attention"], segment_ids=target_segment_ids,
                page_pool=page_pool, max_len=max_len, **sa_kwargs)
        else:
            states, sa = self.self_attention.extend_step(
                cached_states["self_attention"], page_pool=page_pool, **sa_kwargs)
        if sa is None:
            return {"self_attention": states}, None
        x = sa.data
        cross_probs = None
        if cross_attention_data is not None and "cross_attention" in self._children:
            ca = self.cross_attention(target=x, source=cross_attention_data,
                                      attention_logit_biases=cross_attention_logit_biases,
                                      return_aux=return_aux)
            x, cross_probs = ca.data, ca.probs
        if isinstance(x, tuple):
            x = self.feed_forward(x[0], pending_residual=x[1])
        else:
            x = self.feed_forward(x)
        return {"self_attention": states}, self.Output(
            data=x, self_attention_probs=sa.probs, self_attention_kv_state=sa.kv_state,
            cross_attention_probs=cross_probs)

    def forward(self, data, **kwargs):
        # The flag is raised here, inside the (possibly rematerialised) forward, so that the
        # recomputation in the backward pass issues the same collectives.
        sp = self._config.tp_sequence_parallel and coll.axis_size("model") > 1
        with coll.tp_sequence_parallel(sp):
            _, out = self._forward_for_mode(mode=ForwardMode.FORWARD, data=data, **kwargs)
        return out

    def init_states(self, *, time_step, data, page_pool=None, max_len=None, **kwargs):
        if time_step is None:
            states, _ = self.self_attention.init_states(
                time_step=None, target=data, source=kwargs.get("self_attention_kv_state"),
                page_pool=page_pool, max_len=max_len)
            return {"self_attention": states}, None
        return self._forward_for_mode(
            mode=ForwardMode.INIT_STATES, data=data, cached_states={"self_attention": time_step},
            page_pool=page_pool, max_len=max_len, **kwargs)

    def extend_step(self, cached_states, data, *, page_pool=None, **kwargs):
        return self._forward_for_mode(
            mode=ForwardMode.EXTEND_STEP, data=data, cached_states=cached_states,
            page_pool=page_pool, **kwargs)


# ------------------------------------------------------------------------------------------
# Stacks.
# ------------------------------------------------------------------------------------------


class BaseStackedTransformerLayer(BaseTransformerLayer):
    @config_class
    class Config(BaseTransformerLayer.Config):
        num_layers: Required[int] = REQUIRED
        layer: Union[InstantiableConfig, Sequence[InstantiableConfig]] = TransformerLayer.default_config()
        peak_stochastic_depth_rate: Optional[float] = None
        # Sequence-sharded activations between the tensor-parallel blocks (training forward only;
        # see ``TransformerLayer.Config.tp_sequence_parallel``).
        tp_sequence_parallel: bool = False

    def _tp_seq_on(self) -> bool:
        return bool(self._config.tp_sequence_parallel) and coll.axis_size("model") > 1

    def _tp_seq_wrap(self, run, data):
        """Slices the replicated input over the `model` axis, runs the stack on the slice and
        gathers the output (``run(data) -> Output``)."""
        if not self._tp_seq_on():
            return run(data)
        out = run(coll.scatter_replicated(data, "model", dim=1))
        return out._replace(data=coll.gather_replicated(out.data, "model", dim=1))


def _update_data(kwargs: dict, data: Tensor) -> dict:
    return kwargs


class StackedTransformerLayer(BaseStackedTransformerLayer):
    """``num_layers`` separately-parameterised children ``layer0 .. layer{N-1}``."""

    @config_class
    class Config(BaseStackedTransformerLayer.Config):
        # Optional per-layer config hook: (layer_index, layer_cfg) -> layer_cfg.
        layer_config_fn: Optional[Callable] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._layers = []
        layer_cfgs = cfg.layer if isinstance(cfg.layer, (list, tuple)) else [cfg.layer] * cfg.num_layers
        if len(layer_cfgs) != cfg.num_layers:
            raise ValueError("number of layer configs must equal num_layers")
        for i, lc in enumerate(layer_cfgs):
            lc = lc.clone(input_dim=cfg.input_dim)
            if cfg.tp_sequence_parallel and "tp_sequence_parallel" in lc.keys():
                lc.tp_sequence_parallel = True
            if cfg.peak_stochastic_depth_rate:
                rate = cfg.peak_stochastic_depth_rate * (i + 1) / cfg.num_layers
                lc.self_attention.stochastic_depth.rate = rate
                lc.feed_forward.stochastic_depth.rate = rate
            if cfg.layer_config_fn is not None:
                lc = cfg.layer_config_fn(i, lc) or lc
            self._layers.append(self._add_child(f"layer{i}", lc))

    def _forward_for_mode(self, *, mode, data, cached_states=None, return_aux=None, **kwargs):
        all_states = {}
        probs, kvs = [], []
        out = None
        for i, layer in enumerate(self._layers):
            if mode == ForwardMode.FORWARD:
                out = layer(data, return_aux=return_aux, **kwargs)
                st = None
            elif mode == ForwardMode.INIT_STATES:
                st, out = layer.init_states(time_step=cached_states, data=data, return_aux=return_aux, **kwargs)
            else:
                st, out = layer.extend_step(cached_states[layer.name], data, return_aux=return_aux, **kwargs)
            all_states[layer.name] = st
            if out is not None:
                data = out.data
                probs.append(out.self_attention_probs)
                kvs.append(out.self_attention_kv_state)
        if out is None:
            return all_states, None
        return all_states, BaseTransformerLayer.Output(
            data=data,
            self_attention_probs=probs if return_aux and "self_attention_probs" in return_aux else None,
            self_attention_kv_state=kvs if return_aux and "self_attention_kv_state" in return_aux else None,
        )

    def forward(self, data, **kwargs):
        return self._tp_seq_wrap(
            lambda d: self._forward_for_mode(mode=ForwardMode.FORWARD, data=d, **kwargs)[1], data)

    def init_states(self, *, time_step, data, **kwargs):
        return self._forward_for_mode(mode=ForwardMode.INIT_STATES, data=data, cached_states=time_step, **kwargs)

    def extend_step(self, cached_states, data, **kwargs):
        return self._forward_for_mode(mode=ForwardMode.EXTEND_STEP, data=data, cached_states=cached_states, **kwargs)


class _TransformerRepeat(Repeat):
    """Repeat specialised to transformer layers: carries ``data``, threads per-layer cache
    states, and prefetches the next layer's sharded parameters."""

    def forward(self, data, **kwargs):
        def body(carry, _x, layer):
            out = layer(carry, **kwargs)
            return out.data, None

        data, _ = self._run(body, carry=data)
        return data

    def init_states(self, *, time_step, data, **kwargs):
        def body(carry, _x, layer):
            st, out = layer.init_states(time_step=time_step, data=carry, **kwargs)
            return (carry if out is None else out.data), st

        data_out, states = self._run(body, carry=data, collect=True)
        return _as_vdict(states), (None if time_step is None else data_out)

    def extend_step(self, cached_states, data, **kwargs):
        def body(carry, st_i, layer):
            st, out = layer.extend_step(st_i, carry, **kwargs)
            return out.data, st

        data, states = self._run(body, carry=data, xs=cached_states, collect=True)
        return _as_vdict(states), data


def _as_vdict(states):
    """Stacked per-layer states carry the layer dim in front of the batch dim: mark them so that
    batch-wise tree operations (decoding) map over layers."""
    return VDict(states) if isinstance(states, dict) and not isinstance(states, VDict) else states


class RepeatedTransformerLayer(BaseStackedTransformerLayer):
    """One layer config repeated ``num_layers`` times with parameters stacked on a leading
    dim (child ``repeat`` -> ``layer``)."""

    @config_class
    class Config(BaseStackedTransformerLayer.Config):
        repeat: Repeat.Config = _TransformerRepeat.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        layer_cfg = cfg.layer.clone(input_dim=cfg.input_dim)
        if cfg.tp_sequence_parallel and "tp_sequence_parallel" in layer_cfg.keys():
            layer_cfg.tp_sequence_parallel = True
        repeat_cfg = cfg.repeat.clone(layer=layer_cfg, num_layers=cfg.num_layers)
        self._add_child("repeat", repeat_cfg)

    def forward(self, data, *, return_aux=None, **kwargs):
        if return_aux:
            raise NotImplementedError("return_aux is not supported by RepeatedTransformerLayer")
        return self._tp_seq_wrap(lambda d: BaseTransformerLayer.Output(data=self.repeat(d, **kwargs)), data)

    def init_states(self, *, time_step, data, **kwargs):
        kwargs.pop("return_aux", None)
        states, out = self.repeat.init_states(time_step=time_step, data=data, **kwargs)
        return {"repeat": states}, (None if out is None else BaseTransformerLayer.Output(data=out))

    def extend_step(self, cached_states, data, **kwargs):
        kwargs.pop("return_aux", None)
        states, out = self.repeat.extend_step(cached_states["repeat"], data, **kwargs)
        return {"repeat": states}, BaseTransformerLayer.Output(data=out)


# ------------------------------------------------------------------------------------------
# Config helpers.
# ------------------------------------------------------------------------------------------


class RematRegexSavePatterns(enum.Enum):
    QKV_PROJ = r".*[kqv]_proj"
    O_PROJ = r".*o_proj"
    CONTEXT = r".*context"
    LINEAR1_X = r".*linear1_[01]"
    LINEAR2_X = r".*linear2_[01]"
    NATIVE_ATTENTION = ".*([qkvo]_proj|context)"
    FEED_FORWARD = "|".join([LINEAR1_X, LINEAR2_X])
    FLASH_CONTEXT = r".*FlashAttention\.context"
    FLASH_ATTENTION = "|".join([FLASH_CONTEXT, QKV_PROJ, O_PROJ])


save_only_these_names_regex = remat.save_only_these_names_regex
save_and_offload_only_these_names_regex = remat.save_and_offload_only_these_names_regex


def build_remat_spec(
    stack_cfg: ConfigBase,
    save_pattern: Any = RematRegexSavePatterns.NATIVE_ATTENTION.value,
    offload_pattern: Any = None,
    offload_dst: str = "pinned_host",
) -> Optional[RematSpec]:
    """Remat spec for the layers of ``stack_cfg``: tensors tagged with a name matching
    ``save_pattern`` are kept on the device between the first pass and the replay, those matching
    ``offload_pattern`` in pinned host memory, everything else is recomputed (reference:
    axlearn/common/attention.py:4574-4653).  None for pipelined stacks."""
    if getattr(stack_cfg, "klass", None) is not None and stack_cfg.klass.__name__ == "PipelinedTransformerLayer":
        return None
    policy = config_for_function(save_and_offload_only_these_names_regex).set(
        names_which_can_be_saved=save_pattern, names_which_can_be_offloaded=offload_pattern,
        offload_src="device", offload_dst=offload_dst)
    return RematSpec(prevent_cse=False, policy=policy)


def set_double_shard_weights_config(
    cfg: Union[TransformerLayer.Config, Sequence[TransformerLayer.Config]],
    *,
    batch_axis_names: Union[str, Sequence[str]] = ("data", "expert", "fsdp"),
    fsdp_axis_names: Union[str, Sequence[str]] = "fsdp",
    tp_axis_names: Union[str, Sequence[str]] = "model",
    seq_axis_names: Union[str, Sequence[str]] = "seq",
) -> None:
    """Shards transformer weights over both ``fsdp`` (storage) and ``model`` (compute):
    input projections ``(fsdp, model, None)``, output projection ``(fsdp, model, None)``,
    ``linear1*`` ``(fsdp, model)``, ``linear2`` ``(model, fsdp)``."""
    del batch_axis_names, seq_axis_names

    def set_attn(attn_cfg):
        il = attn_cfg.input_linear
        if "input_linear" in il:
            il = il.input_linear
        il.layer.param_partition_spec = (
            (None, fsdp_axis_names, tp_axis_names, None)
            if il.klass is FusedQKVLinear and il.layer.klass is _FusedQKVProj
            else (fsdp_axis_names, tp_axis_names, None)
        )
        attn_cfg.output_linear.param_partition_spec = (fsdp_axis_names, tp_axis_names, None)

    def _as_tuple(a):
        return (a,) if isinstance(a, str) else tuple(a)

    def set_ffn(ff_cfg):
        ff_cfg.linear1.param_partition_spec = (fsdp_axis_names, tp_axis_names)
        # The reference shards linear2 as (model, fsdp), i.e. storage-sharded on its *output*
        # columns.  Here every storage shard is a contiguous row-slab (what the in-kernel
        # all-gather and the reduce-scatter epilogue move), so linear2's rows are split over
        # model (major) and then the storage axes; the global shape is unchanged.
        ff_cfg.linear2.param_partition_spec = (_as_tuple(tp_axis_names) + _as_tuple(fsdp_axis_names), None)

    for layer_cfg in cfg if isinstance(cfg, (list, tuple)) else [cfg]:
        set_attn(layer_cfg.self_attention.attention)
        if layer_cfg.cross_attention is not None:
            set_attn(layer_cfg.cross_attention.attention)
        if "linear1" in layer_cfg.feed_forward:
            set_ffn(layer_cfg.feed_forward)
