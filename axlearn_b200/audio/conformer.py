"""Conformer blocks.

Parity targets in the reference (axlearn/common/conformer.py): ``LConvLayer`` (:60-170: norm ->
pointwise linear to 2x dim -> GLU -> depthwise conv over time -> norm -> activation -> pointwise
linear -> dropout, residual) and ``ConformerLayer`` (:230-420: half-step feed-forward -> self
attention -> convolution module -> half-step feed-forward -> final layer norm; paddings zeroed
between the parts), ``RepeatedConformerLayer`` (:540).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.attention import MultiheadAttention, TransformerAttentionLayer, TransformerFeedForwardLayer
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import DepthwiseConv1D
from axlearn_b200.common.layers import BatchNorm, Dropout, LayerNorm, Linear, get_activation_fn

Tensor = torch.Tensor
NEG_INF = -1e9


class LConvLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        linear1: InstantiableConfig = Linear.default_config().set(bias=True)
        conv: InstantiableConfig = DepthwiseConv1D.default_config().set(window=15, padding="SAME", bias=False)
        conv_norm: InstantiableConfig = LayerNorm.default_config()
        conv_activation: str = "nn.silu"
        linear2: InstantiableConfig = Linear.default_config().set(bias=True)
        norm: InstantiableConfig = LayerNorm.default_config()
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        d = cfg.input_dim
        self._add_child("norm", cfg.norm.clone(input_dim=d))
        self._add_child("linear1_0", cfg.linear1.clone(input_dim=d, output_dim=d))
        self._add_child("linear1_1", cfg.linear1.clone(input_dim=d, output_dim=d))
        self._add_child("conv", cfg.conv.clone(input_dim=d))
        self._add_child("conv_norm", cfg.conv_norm.clone(input_dim=d))
        self._add_child("linear2", cfg.linear2.clone(input_dim=d, output_dim=d))
        self._add_child("dropout", cfg.dropout)

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        live = (1 - paddings)[..., None].to(inputs.dtype)
        x = self.norm(inputs)
        x = self.linear1_0(x) * torch.sigmoid(self.linear1_1(x))          # GLU
        x = self.conv(x * live)
        x = get_activation_fn(self._config.conv_activation)(self.conv_norm(x))
        x = self.dropout(self.linear2(x))
        return inputs + x * live


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
    """``num_layers`` conformer layers in sequence (children ``layer{i}``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_layers: Required[int] = REQUIRED
        layer: InstantiableConfig = ConformerLayer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._layers = [self._add_child(f"layer{i}", cfg.layer.clone(input_dim=cfg.input_dim))
                        for i in range(cfg.num_layers)]

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        x = inputs
        for layer in self._layers:
            x = layer(x, paddings=paddings)
        return x
