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
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class, config_for_function
from axlearn_b200.common.encoder import NEG_INF, Encoder, _padding_bias

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
    """Per-head logit bias by bucketed relative position (child ``emb``: an embedding table
    ``[num_buckets, dim]`` with ``dim`` = number of heads)."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED          # number of attention heads
        num_buckets: int = 32
        max_distance: int = 128
        bidirectional: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        from axlearn_b200.common.layers import Embedding
        from axlearn_b200.common.param_init import DefaultInitializer, WeightInitializer

        init = DefaultInitializer.default_config().set(init_by_param_name={
            ".*weight$": WeightInitializer.default_config().set(fan="fan_avg", distribution="uniform", scale=1.0)})
        self._add_child("emb", Embedding.default_config().set(num_embeddings=cfg.num_buckets, dim=cfg.dim, param_init=init))

    def forward(self, query_len: int, key_len: Optional[int] = None, *, device=None) -> Tensor:
        """``[1, num_heads, query_len, key_len]`` additive logit biases."""
        cfg = self._config
        key_len = key_len or query_len
        q = torch.arange(query_len, device=device)[:, None]
        k = torch.arange(key_len, device=device)[None, :]
        buckets = t5_relative_position_bucket(k - q, bidirectional=cfg.bidirectional, num_buckets=cfg.num_buckets,
                                              max_distance=cfg.max_distance)
        bias = self.emb(buckets)                                                           # [T, S, N]
        return bias.permute(2, 0, 1)[None]


class EncoderOutputLayer(BaseLayer):
    """Final norm + dropout of the encoder (children ``norm`` and ``dropout``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        norm: InstantiableConfig = None
        dropout: InstantiableConfig = None

    @classmethod
    def default_config(cls):
        from axlearn_b200.common.layers import Dropout, RMSNorm

        cfg = super().default_config()
        cfg.norm = RMSNorm.default_config()
        cfg.dropout = Dropout.default_config()
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("norm", cfg.norm.clone(input_dim=cfg.input_dim))
        self._add_child("dropout", cfg.dropout)

    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(self.norm(x))


def t5_transformer_stack_config(arch: str = "t5-v1-1", hidden_dim=None, base_cfg=None):
    """Pre-norm layers without biases; feed-forward by architecture: ``t5-v1-1`` gated GELU of
    width 8/3, ``t5-v1`` ReLU of width 4, ``t5-ul2`` gated SiLU of width 8/3."""
    from axlearn_b200.common.attention import StackedTransformerLayer, scaled_hidden_dim
    from axlearn_b200.common.layers import set_bias_recursively

    cfg = base_cfg or StackedTransformerLayer.default_config()
    cfg.layer.feed_forward.set(structure="prenorm")
    if arch == "t5-v1-1":
        cfg.layer.feed_forward.set(activation=("nn.gelu", "linear"), hidden_dim=scaled_hidden_dim(8.0 / 3))
    elif arch == "t5-v1":
        cfg.layer.feed_forward.set(activation="nn.relu", hidden_dim=scaled_hidden_dim(4))
    elif arch == "t5-ul2":
        cfg.layer.feed_forward.set(activation=("nn.silu", "linear"), hidden_dim=scaled_hidden_dim(8.0 / 3))
    else:
        raise ValueError(f"Unsupported arch {arch}.")
    if hidden_dim is not None:
        cfg.layer.feed_forward.set(hidden_dim=hidden_dim)
    set_bias_recursively(cfg, False)
    return cfg


class T5Encoder(Encoder):
    """``Encoder`` whose self-attention logits get the shared relative position bias (reference:
    axlearn/common/t5.py ``T5Encoder``).  With ``causal=True`` it is a decoder-side self-attention
    stack (one-sided buckets + causal mask)."""

    @config_class
    class Config(Encoder.Config):
        relative_pos_emb: InstantiableConfig = T5RelativePositionalEmbedding.default_config()
        causal: bool = False

    @classmethod
    def default_config(cls):
        from axlearn_b200.common.embedding import TransformerTextEmbeddings
        from axlearn_b200.common.layers import RMSNorm, set_norm_recursively

        cfg = super().default_config()
        cfg.emb = TransformerTextEmbeddings.default_config().set(pos_emb=None)
        cfg.transformer = t5_transformer_stack_config()
        cfg.output = EncoderOutputLayer.default_config()
        cfg.pad_token_id = 0
        set_norm_recursively(cfg, RMSNorm.default_config())
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("relative_pos_emb", cfg.relative_pos_emb.clone(bidirectional=not cfg.causal))

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


def t5_encoder_config(*, vocab_size: int, dim: int, num_layers: int, num_attention_heads: int,
                      ffn_dim: Optional[int] = None, arch: str = "t5-v1-1", causal: bool = False,
                      dropout_rate: float = 0.0, base_cfg: Optional[InstantiableConfig] = None) -> "T5Encoder.Config":
    """RMSNorm pre-norm layers, no biases, no absolute positions, shared relative position bias.
    (As in the reference the attention keeps its ``1 / sqrt(head_dim)`` query scale; converters
    from T5X checkpoints fold the difference into the query weights.)"""
    from axlearn_b200.common.layers import RMSNorm, set_bias_recursively, set_dropout_rate_recursively, set_norm_recursively

    cfg = base_cfg.clone() if base_cfg is not None else T5Encoder.default_config()
    cfg.set(vocab_size=vocab_size, dim=dim, causal=causal)
    cfg.transformer = t5_transformer_stack_config(arch, hidden_dim=ffn_dim, base_cfg=cfg.transformer)
    cfg.relative_pos_emb.dim = num_attention_heads
    cfg.transformer.set(num_layers=num_layers)
    cfg.transformer.layer.self_attention.attention.num_heads = num_attention_heads
    set_bias_recursively(cfg, False)
    set_norm_recursively(cfg, RMSNorm.default_config())
    if dropout_rate:
        set_dropout_rate_recursively(cfg, dropout_rate)
    return cfg


# ------------------------------------------------------------------------------------------
# Decoder and encoder-decoder (reference: axlearn/common/t5.py ``t5_decoder_config``,
# ``t5_encoder_decoder_config``).
# ------------------------------------------------------------------------------------------


class T5DecoderLogitBias(BaseLayer):
    """The decoder's self-attention bias as a ``Decoder.attention_mask`` layer: causal and segment
    masks plus the one-sided relative position bias shared by all layers (child
    ``relative_pos_emb``).  Being a function of positions it serves training, prefill and
    single-step decoding alike."""

    @config_class
    class Config(BaseLayer.Config):
        num_heads: Required[int] = REQUIRED
        relative_pos_emb: InstantiableConfig = T5RelativePositionalEmbedding.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("relative_pos_emb", cfg.relative_pos_emb.clone(dim=cfg.num_heads, bidirectional=False))

    def forward(self, *, segment_ids: Tensor, positions: Tensor) -> Tensor:
        rel_cfg = self._config.relative_pos_emb
        rel = positions[:, None, :] - positions[:, :, None]                       # key - query
        buckets = t5_relative_position_bucket(rel, bidirectional=False, num_buckets=rel_cfg.num_buckets,
                                              max_distance=rel_cfg.max_distance)
        bias = self.relative_pos_emb.emb(buckets).permute(0, 3, 1, 2).float()     # [B, N, T, S]
        ok = (rel <= 0) & (segment_ids[:, :, None] == segment_ids[:, None, :])
        return bias + torch.where(ok, 0.0, NEG_INF)[:, None]


def t5_decoder_config(*, vocab_size: int, dim: int, num_layers: int, num_attention_heads: int,
                      ffn_dim: Optional[int] = None, arch: str = "t5-v1-1", dropout_rate: float = 0.0):
    """A ``Decoder`` with cross-attention; ``t5-v1`` ties the output head to the embedding (logits
    scaled by ``dim ** -0.5``), the later architectures have their own ``lm_head``."""
    from axlearn_b200.common.attention import TransformerAttentionLayer
    from axlearn_b200.common.decoder import Decoder, LmHead
    from axlearn_b200.common.embedding import TransformerTextEmbeddings
    from axlearn_b200.common.layers import RMSNorm, set_bias_recursively, set_dropout_rate_recursively, set_norm_recursively

    cfg = Decoder.default_config().set(vocab_size=vocab_size, dim=dim, pad_token_id=0, eos_token_id=1)
    cfg.emb = TransformerTextEmbeddings.default_config().set(pos_emb=None)
    cfg.transformer = t5_transformer_stack_config(arch, hidden_dim=ffn_dim)
    cfg.transformer.set(num_layers=num_layers)
    layer = cfg.transformer.layer
    layer.self_attention.attention.num_heads = num_attention_heads
    layer.cross_attention = TransformerAttentionLayer.default_config().set(source_dim=dim)
    layer.cross_attention.attention.num_heads = num_attention_heads
    cfg.attention_mask = T5DecoderLogitBias.default_config().set(num_heads=num_attention_heads)
    if arch == "t5-v1":
        from axlearn_b200.common import logit_modifiers  # pylint: disable=import-outside-toplevel

        cfg.output_logits_modifier = config_for_function(logit_modifiers.scale_by).set(temperature=dim ** 0.5)
    else:
        cfg.lm_head = LmHead.default_config()
    set_bias_recursively(cfg, False)
    set_norm_recursively(cfg, RMSNorm.default_config())
    cfg.output_norm = RMSNorm.default_config()
    if dropout_rate:
        set_dropout_rate_recursively(cfg, dropout_rate)
    return cfg


def t5_encoder_decoder_config(*, vocab_size: int, dim: int, num_attention_heads: int, num_encoder_layers: int,
                              num_decoder_layers: int, ffn_dim: Optional[int] = None, arch: str = "t5-v1-1",
                              dropout_rate: float = 0.0):
    from axlearn_b200.common.encoder import EncoderDecoderModel

    kw = dict(vocab_size=vocab_size, dim=dim, num_attention_heads=num_attention_heads, ffn_dim=ffn_dim, arch=arch,
              dropout_rate=dropout_rate)
    return EncoderDecoderModel.default_config().set(
        encoder=t5_encoder_config(num_layers=num_encoder_layers, **kw),
        decoder=t5_decoder_config(num_layers=num_decoder_layers, **kw))
