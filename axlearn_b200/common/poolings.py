"""Pooling over the sequence dim of ``[B, T, D]`` token representations.

Parity targets in the reference (axlearn/common/poolings.py): ``AveragePooling``, ``MaxPooling``,
``FirstNTokenPooling``, ``LastNTokenPooling``, ``AttentionPooling`` -- all map
``(tokens [B, T, D], paddings [B, T]) -> [B, num_outputs, D]``.
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.attention import MultiheadAttention
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import LayerNorm
from axlearn_b200.common.param_init import gaussian_initializer

Tensor = torch.Tensor


class BasePoolingLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        num_outputs: int = 1

    def forward(self, tokens: Tensor, paddings: Optional[Tensor] = None) -> Tensor:
        raise NotImplementedError(type(self))


def _live(tokens: Tensor, paddings: Optional[Tensor]) -> Tensor:
    if paddings is None:
        return torch.ones(tokens.shape[:2], dtype=torch.bool, device=tokens.device)
    return paddings == 0


class AveragePooling(BasePoolingLayer):
    def forward(self, tokens, paddings=None):
        live = _live(tokens, paddings)[..., None].to(tokens.dtype)
        return ((tokens * live).sum(dim=1) / live.sum(dim=1).clamp_min(1.0))[:, None, :]


class MaxPooling(BasePoolingLayer):
    def forward(self, tokens, paddings=None):
        live = _live(tokens, paddings)[..., None]
        masked = tokens.masked_fill(~live, torch.finfo(tokens.dtype).min)
        out = masked.amax(dim=1)
        return torch.where(live.any(dim=1), out, torch.zeros_like(out))[:, None, :]


class FirstNTokenPooling(BasePoolingLayer):
    def forward(self, tokens, paddings=None):
        return tokens[:, :self._config.num_outputs]


class LastNTokenPooling(BasePoolingLayer):
    """The last ``num_outputs`` non-padding tokens of every row (zeros when a row is shorter)."""

    def forward(self, tokens, paddings=None):
        n = self._config.num_outputs
        live = _live(tokens, paddings)
        lengths = live.sum(dim=1)
        idx = lengths[:, None] - n + torch.arange(n, device=tokens.device)[None]
        ok = idx >= 0
        out = torch.gather(tokens, 1, idx.clamp_min(0)[..., None].expand(-1, -1, tokens.shape[-1]))
        return out * ok[..., None].to(out.dtype)


class AttentionPooling(BasePoolingLayer):
    """``num_outputs`` learned queries attend over the tokens (CoCa-style)."""

    @config_class
    class Config(BasePoolingLayer.Config):
        num_heads: int = 1
        cross_attention: InstantiableConfig = MultiheadAttention.default_config()
        norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("cross_attention", cfg.cross_attention.clone(
            query_dim=cfg.output_dim, key_dim=cfg.input_dim, value_dim=cfg.input_dim, output_dim=cfg.output_dim,
            num_heads=cfg.num_heads))
        self._add_child("norm", cfg.norm.clone(input_dim=cfg.output_dim))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"query": ParameterSpec(shape=(cfg.num_outputs, cfg.output_dim), mesh_axes=(None, None),
                                       initializer=gaussian_initializer(cfg.output_dim ** -0.5))}

    def forward(self, tokens, paddings=None):
        b = tokens.shape[0]
        q = self.parameters["query"].to(tokens.dtype)[None].expand(b, -1, -1)
        bias = None
        if paddings is not None:
            bias = torch.where(paddings[:, None, None, :] == 0, 0.0, -1e9).to(tokens.dtype)
        out = self.cross_attention(q, key=tokens, value=tokens, attention_logit_biases=bias)
        return self.norm(out.data)
