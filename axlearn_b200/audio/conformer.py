"""Conformer blocks.

Parity targets in the reference (axlearn/common/conformer.py): ``LConvLayer`` (:60-170: norm ->
gated linear unit -> depthwise conv over time -> batch norm -> activation -> pointwise linear ->
dropout, residual) and ``ConformerLayer`` (:230-420: half-step feed-forward -> relative-position
self attention (``MultiheadAttentionXL``) -> convolution module -> half-step feed-forward -> final
layer norm; paddings zeroed between the parts), ``RepeatedConformerLayer`` (:540, stacked
parameters under ``repeat/layer``).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.attention import MultiheadAttention, TransformerAttentionLayer, TransformerFeedForwardLayer
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import DepthwiseConv1D
from axlearn_b200.common.layers import BatchNorm, Dropout, LayerNorm, Linear, get_activation_fn
from axlearn_b200.common.repeat import Repeat

Tensor = torch.Tensor
NEG_INF = -1e9


class LConvLayer(BaseLayer):
    """The convolution module: ``linear1_norm`` -> gated linear unit (``linear1_0`` x
    ``sigmoid(linear1_1)``) -> depthwise ``conv`` over time -> ``conv_norm`` (batch norm) ->
    activation -> ``linear2`` -> dropout, with a residual connection."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        linear1_norm: InstantiableConfig = LayerNorm.default_config()
        linear1_activation: tuple = ("linear", "nn.sigmoid")
        linear1: InstantiableConfig = Linear.default_config().set(bias=True)
        conv: InstantiableConfig = DepthwiseConv1D.default_config().set(window=32, padding="SAME", bias=False)
        conv_norm: InstantiableConfig = BatchNorm.default_config()
        conv_activation: str = "nn.silu"
        linear2: InstantiableConfig = Linear.default_config().set(bias=True)
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        d = cfg.input_dim
        self._add_child("linear1_norm", cfg.linear1_norm.clone(input_dim=d))
        self._add_child("linear1_0", cfg.linear1.clone(input_dim=d, output_dim=d))
        self._add_child("linear1_1", cfg.linear1.clone(input_dim=d, output_dim=d))
        self._add_child("conv", cfg.conv.clone(input_dim=d))
        self._add_child("conv_norm", cfg.conv_norm.clone(input_dim=d))
        self._add_child("linear2", cfg.linear2.clone(input_dim=d, output_dim=d))
        self._add_child("dropout", cfg.dropout)

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        cfg = self._config
        live = (1 - paddings)[..., None].to(inputs.dtype)
        x = self.linear1_norm(inputs)
        a0, a1 = (get_activation_fn(a) for a in cfg.linear1_activation)
        x = a0(self.linear1_0(x)) * a1(self.linear1_1(x))
        x = self.conv(x * live)
        x = get_activation_fn(cfg.conv_activation)(self.conv_norm(x, paddings=paddings))
        x = self.dropout(self.linear2(x))
        return inputs + x * live


def _xl_attention_config():
    """Relative-position self-attention of the conformer: Transformer-XL logits, scale (with a
    learned per-dim factor) applied to the query, fused biased QKV projection."""
    from axlearn_b200.common.attention import FusedQKVLinear, PerDimScale
    from axlearn_b200.common.attention_xl import MultiheadAttentionXL

    cfg = MultiheadAttentionXL.default_config().set(scale_position=MultiheadAttentionXL.ScalePosition.QUERY)
    cfg.input_linear = FusedQKVLinear.default_config()
    cfg.input_linear.layer.bias = True
    cfg.query_scale.per_dim_scale = PerDimScale.default_config()
    return cfg


class ConformerLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_heads: int = 4
        ff_start: InstantiableConfig = TransformerFeedForwardLayer.default_config().set(
            activation="nn.silu", residual_weight=0.5)
        self_attention: InstantiableConfig = TransformerAttentionLayer.default_config()
        lconv: InstantiableConfig = LConvLayer.default_config()
        ff_end: InstantiableConfig = TransformerFeedForwardLayer.default_config().set(
            activation="nn.silu", residual_weight=0.5)
        norm: InstantiableConfig = LayerNorm.default_config()
        ff_hidden_scale: int = 4
        # Attention window (frames to the left / right); None = the whole utterance.
        left_context: Optional[int] = None
        right_context: Optional[int] = None

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.self_attention.attention = _xl_attention_config()
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        d = cfg.input_dim
        self._add_child("ff_start", cfg.ff_start.clone(input_dim=d, hidden_dim=d * cfg.ff_hidden_scale))
        att = cfg.self_attention.clone(target_dim=d, source_dim=d)
        att.attention.num_heads = cfg.num_heads
        self._add_child("self_attention", att)
        self._add_child("lconv", cfg.lconv.clone(input_dim=d))
        self._add_child("ff_end", cfg.ff_end.clone(input_dim=d, hidden_dim=d * cfg.ff_hidden_scale))
        self._add_child("norm", cfg.norm.clone(input_dim=d))

    def _attention_bias(self, paddings: Tensor, dtype) -> Tensor:
        cfg = self._config
        t = paddings.shape[1]
        bias = torch.where(paddings[:, None, None, :] > 0, NEG_INF, 0.0).to(dtype)
        if cfg.left_context is not None or cfg.right_context is not None:
            pos = torch.arange(t, device=paddings.device)
            rel = pos[None, :] - pos[:, None]                     # key - query
            ok = torch.ones(t, t, dtype=torch.bool, device=paddings.device)
            if cfg.left_context is not None:
                ok &= rel >= -cfg.left_context
            if cfg.right_context is not None:
                ok &= rel <= cfg.right_context
            bias = bias + torch.where(ok, 0.0, NEG_INF).to(dtype)[None, None]
        return bias

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        live = (1 - paddings)[..., None].to(inputs.dtype)
        x = self.ff_start(inputs) * live
        x = self.self_attention(target=x, attention_logit_biases=self._attention_bias(paddings, x.dtype)).data * live
        x = self.lconv(x, paddings=paddings)
        x = self.ff_end(x) * live
        return self.norm(x) * live


class RepeatedConformerLayer(BaseLayer):
    """``num_layers`` conformer layers with parameters stacked on a leading dim (child ``repeat``
    -> ``layer``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_layers: Required[int] = REQUIRED
        layer: InstantiableConfig = ConformerLayer.default_config()
        repeat: InstantiableConfig = Repeat.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("repeat", cfg.repeat.clone(layer=cfg.layer.clone(input_dim=cfg.input_dim),
                                                   num_layers=cfg.num_layers))

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        return self.repeat(inputs, paddings=paddings)
