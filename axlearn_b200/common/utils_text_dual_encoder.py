"""Builders for text dual encoders: a BERT tower config and initial-state builders.

Counterpart of axlearn/common/utils_text_dual_encoder.py (``bert_text_embedding_stream_encoder_config``
:31, ``init_state_builder_config`` :107, ``init_state_builder_siamese_model_config`` :146).
"""

from __future__ import annotations

from typing import Optional

from axlearn_b200.common.attention import RepeatedTransformerLayer, StackedTransformerLayer
from axlearn_b200.common.config import InstantiableConfig
from axlearn_b200.common.encoder import Encoder, bert_embedding_config, bert_transformer_config
from axlearn_b200.common.layers import L2Norm, Linear, set_dropout_rate_recursively
from axlearn_b200.common.poolings import FirstNTokenPooling
from axlearn_b200.common.state_builder import ChainBuilder, RestoreAndConvertBuilder
from axlearn_b200.common.text_dual_encoder import TextEmbeddingStreamEncoder
from axlearn_b200.common.text_encoder import TextEmbeddingEncoder

_DEFAULT = object()


def bert_text_embedding_stream_encoder_config(
        *, pad_token_id: int, vocab_size: int, max_seq_len: int, num_layers: int, num_heads: int, hidden_dim: int,
        output_dim: int, output_proj=_DEFAULT, output_norm=_DEFAULT, pooler: Optional[InstantiableConfig] = None,
        remat: bool = False) -> InstantiableConfig:
    """A BERT encoder (token, position and type embeddings; dropout 0.1) whose first-token state is
    projected (``Linear`` with bias by default) and L2-normalised (by default)."""
    if output_proj is _DEFAULT:
        output_proj = Linear.default_config().set(bias=True)
    if output_norm is _DEFAULT:
        output_norm = L2Norm.default_config()
    base = (RepeatedTransformerLayer if remat else StackedTransformerLayer).default_config()
    encoder = Encoder.default_config().set(
        vocab_size=vocab_size,
        emb=bert_embedding_config(max_position_embeddings=max_seq_len, type_vocab_size=2, layer_norm_epsilon=1e-12),
        transformer=bert_transformer_config(num_layers=num_layers, num_heads=num_heads, layer_norm_epsilon=1e-12,
                                            base_cfg=base))
    set_dropout_rate_recursively(encoder, 0.1)
    return TextEmbeddingStreamEncoder.default_config().set(
        text_encoder=TextEmbeddingEncoder.default_config().set(
            pad_token_id=pad_token_id, encoder=encoder, pooler=pooler or FirstNTokenPooling.default_config()),
        output_dim=output_dim, output_proj=output_proj, output_norm=output_norm, hidden_dim=hidden_dim)


def init_state_builder_config(*, left_encoder_init_state_builder: Optional[InstantiableConfig] = None,
                              right_encoder_init_state_builder: Optional[InstantiableConfig] = None,
                              converter: Optional[InstantiableConfig] = None) -> Optional[InstantiableConfig]:
    """Chains the towers' builders (each restores its own tower), optionally through a converter."""
    builders = [b for b in (left_encoder_init_state_builder, right_encoder_init_state_builder) if b is not None]
    if not builders:
        return None
    chain = ChainBuilder.default_config().set(builders=builders)
    if converter is None:
        return chain
    return RestoreAndConvertBuilder.default_config().set(builder=chain, converter=converter)


def init_state_builder_siamese_model_config(*, shared_encoder_init_state_builder: Optional[InstantiableConfig] = None,
                                            converter: Optional[InstantiableConfig] = None) -> Optional[InstantiableConfig]:
    if shared_encoder_init_state_builder is None:
        return None
    if converter is None:
        return shared_encoder_init_state_builder
    return RestoreAndConvertBuilder.default_config().set(builder=shared_encoder_init_state_builder, converter=converter)
