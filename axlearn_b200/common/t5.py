"""T5-style relative position biases and encoder.

Parity targets in the reference: ``T5RelativePositionalEmbedding`` (axlearn/common/
attention.py:720-840: relative distances are mapped to ``num_buckets`` buckets -- exact for small
distances, logarithmic up to ``max_distance`` -- and every (bucket, head) has a learned scalar
added to the attention logits; bidirectional for encoders, one-sided for decoders) and the T5
builders of axlearn/common/t5.py (pre-norm RMSNorm without bias, no absolute positions, the
first layer's bias table shared by all layers, logits not scaled by ``1/sqrt(d)``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.encoder import NEG_INF, Encoder, _padding_bias
from axlearn_b200.common.param_init import gaussian_initializer

Tensor = torch.Tensor


def t5_relative_position_bucket(relative_position: Tensor, *, bidirectional: bool, num_buckets: int = 32,
                                max_distance: int = 128) -> Tensor:
    """``relative_position = key_position - query_position`` -> bucket ids in ``[0, num_buckets)``."""
    rp = relative_position.long()
    buckets = torch.zeros_like(rp)
    n = num_buckets
    if bidirectional:
        n //= 2
        buckets = buckets + (rp > 0).long() * n
        rp = rp.abs()
    else:
        rp = (-rp).clamp_min(0)
    max_exact = n // 2
    is_small = rp < max_exact
    large = max_exact + (torch.log(rp.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (n - max_exact)).long()
    large = large.clamp(max=n - 1)
    return buckets + torch.where(is_small, rp, large)


class T5RelativePositionalEmbedding(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        num_heads: Required[int] = REQUIRED
        num_buckets: int = 32
        max_distance: int = 128
        bidirectional: bool = True

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"weight": ParameterSpec(shape=(cfg.num_buckets, cfg.num_heads), mesh_axes=(None, "model"),
                                        initializer=gaussian_initializer(1.0))}

    def forward(self, query_len: int, key_len: Optional[int] = None, *, device=None) -> Tensor:
        """``[1, num_heads, query_len, key_len]`` additive logit biases."""
        cfg = self._config
        key_len = key_len or query_len
        q = torch.arange(query_len, device=device)[:, None]
        k = torch.arange(key_len, device=device)[None, :]
        buckets = t5_relative_position_bucket(k - q, bidirectional=cfg.bidirectional, num_buckets=cfg.num_buckets,
                                              max_distance=cfg.max_distance)
        bias = self.parameters["weight"][buckets.to(self.parameters["weight"].device)]     # [T, S, N]
        return bias.permute(2, 0, 1)[None]


class T5Encoder(Encoder):
    """``Encoder`` whose self-attention logits get the shared relative position bias.  With
    ``causal=True`` it is the decoder-side self-attention stack (one-sided buckets + causal mask)."""

    @config_class
    class Config(Encoder.Config):
        relative_pos_emb: InstantiableConfig = T5RelativePositionalEmbedding.default_config()
        num_heads: Required[int] = REQUIRED
        causal: bool = False

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("relative_pos_emb", cfg.relative_pos_emb.clone(
            num_heads=cfg.num_heads, bidirectional=not cfg.causal))

    def forward(self, input_ids: Tensor, **kwargs) -> Tensor:
        cfg = self._config
        live = input_ids != cfg.pad_token_id
        x = self.emb({"inputs": input_ids, "token_type_ids": kwargs.get("token_type_ids"),
                      "positions": kwargs.get("positions")})
        t = input_ids.shape[1]
        bias = _padding_bias(live, x.dtype) + self.relative_pos_emb(t, device=input_ids.device).to(x.dtype)
        if cfg.causal:
            causal = torch.tril(torch.ones(t, t, dtype=torch.bool, device=input_ids.device))
            bias = bias + torch.where(causal[None, None], 0.0, NEG_INF).to(x.dtype)
        x = self.transformer(x, self_attention_logit_biases=bias).data
        if "output" in self._children:
            x = self.output(x)
        return self.output_dropout(x)


def t5_encoder_config(*, vocab_size: int, dim: int, num_layers: int, num_heads: int, ffn_dim: Optional[int] = None,
                      causal: bool = False, dropout_rate: float = 0.0) -> T5Encoder.Config:
    """T5 v1.1 block structure: RMSNorm pre-norm, gated-GELU feed-forward, no biases, unscaled
    attention logits, no absolute position embeddings."""
    from axlearn_b200.common.attention import StackedTransformerLayer, constant_scale_fn
    from axlearn_b200.common.config import config_for_function
    from axlearn_b200.common.embedding import TransformerTextEmbeddings
    from axlearn_b200.common.layers import RMSNorm, set_bias_recursively, set_dropout_rate_recursively, set_norm_recursively

    cfg = T5Encoder.default_config().set(vocab_size=vocab_size, dim=dim, num_heads=num_heads, causal=causal)
    cfg.emb = TransformerTextEmbeddings.default_config().set(pos_emb=None)
    cfg.transformer = StackedTransformerLayer.default_config().set(num_layers=num_layers)
    layer = cfg.transformer.layer
    layer.self_attention.attention.num_heads = num_heads
    layer.self_attention.attention.query_scale.scale_factor = config_for_function(constant_scale_fn).set(value=1.0)
    layer.feed_forward.set(hidden_dim=ffn_dim or 4 * dim, activation=("nn.gelu", "linear"))
    cfg.output = RMSNorm.default_config().set(eps=1e-6)
    set_norm_recursively(cfg, RMSNorm.default_config().set(eps=1e-6))
    set_bias_recursively(cfg, False)
    set_dropout_rate_recursively(cfg, dropout_rate)
    return cfg
