"""Layers that turn ``(segment_ids, positions)`` into attention logit biases.

Reference: axlearn/common/attention.py (``AttentionLogitBiasLayer`` family and
``alibi_get_slopes`` :4719, ``ALiBiAttentionLogitBiasLayer`` :4749,
``SymmetricALiBiAttentionLogitBiasLayer`` :4785).  A decoder with ``attention_mask`` set passes the
layer's output to every self-attention layer as ``self_attention_logit_biases``.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, Required, config_class

Tensor = torch.Tensor
NEG_INF = -1e15


def alibi_get_slopes(num_heads: int) -> list:
    """Head ``h`` of ``n = 2^k`` heads has slope ``2^(-8 (h + 1) / n)``; other head counts take the
    slopes of the power of two below and every other slope of the one above."""

    def power_of_2(n: int) -> list:
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]

    if math.log2(num_heads).is_integer():
        return power_of_2(num_heads)
    below = 2 ** math.floor(math.log2(num_heads))
    return power_of_2(below) + alibi_get_slopes(2 * below)[0::2][: num_heads - below]


class AttentionLogitBiasLayer(BaseLayer):
    """``forward(segment_ids [B, T], positions [B, T]) -> [B, 1 or heads, T, T]``."""

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        raise NotImplementedError(type(self))


def _segment_bias(segment_ids: Tensor) -> Tensor:
    same = segment_ids[:, :, None] == segment_ids[:, None, :]
    return torch.where(same, 0.0, NEG_INF)[:, None]


class FullAttentionLogitBiasLayer(AttentionLogitBiasLayer):
    """Every position attends to every position of its own segment."""

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        return _segment_bias(segment_ids)


class CausalAttentionLogitBiasLayer(AttentionLogitBiasLayer):
    """... and only to positions at or before its own."""

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        causal = positions[:, :, None] >= positions[:, None, :]
        return _segment_bias(segment_ids) + torch.where(causal, 0.0, NEG_INF)[:, None]


class ALiBiAttentionLogitBiasLayer(CausalAttentionLogitBiasLayer):
    """Causal bias plus ``slope_h * (key position - query position)``."""

    @config_class
    class Config(CausalAttentionLogitBiasLayer.Config):
        num_heads: Required[int] = REQUIRED

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        slopes = torch.tensor(alibi_get_slopes(self._config.num_heads), device=positions.device)
        rel = (positions[:, None, :] - positions[:, :, None]).float()[:, None]          # key - query
        bias = rel * slopes[None, :, None, None]
        return (bias + super().forward(segment_ids=segment_ids, positions=positions)).clamp_min(NEG_INF)


class SymmetricALiBiAttentionLogitBiasLayer(FullAttentionLogitBiasLayer):
    """Bidirectional ALiBi: ``-slope_h * |key position - query position|``."""

    @config_class
    class Config(FullAttentionLogitBiasLayer.Config):
        num_heads: Required[int] = REQUIRED

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        slopes = -torch.tensor(alibi_get_slopes(self._config.num_heads), device=positions.device)
        rel = (positions[:, None, :] - positions[:, :, None]).abs().float()[:, None]
        bias = rel * slopes[None, :, None, None]
        return (bias + super().forward(segment_ids=segment_ids, positions=positions)).clamp_min(NEG_INF)


def decode_step_bias(layer: AttentionLogitBiasLayer, *, query_positions: Tensor, key_len: int) -> Tensor:
    """Rows of the ``[key_len, key_len]`` bias at ``query_positions [B, steps]`` (one segment):
    what a decoding step at those positions sees of a cache of ``key_len`` slots."""
    b = query_positions.shape[0]
    positions = torch.arange(key_len, device=query_positions.device)[None].expand(b, -1)
    full = layer(segment_ids=torch.ones_like(positions), positions=positions)          # [B, H, L, L]
    idx = query_positions.clamp(0, key_len - 1).long()[:, None, :, None].expand(-1, full.shape[1], -1, key_len)
    return torch.gather(full, 2, idx)
