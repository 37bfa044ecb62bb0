"""DistilBERT as a text embedding encoder.

Reference: axlearn/common/distilbert.py:28-106 (``set_distilbert_config``): a 6-layer BERT
encoder without token-type embeddings and a first-token pooler; defaults follow the Hugging
Face release.
"""

from __future__ import annotations

from typing import Optional, Union

from axlearn_b200.common.attention import RepeatedTransformerLayer, StackedTransformerLayer, scaled_hidden_dim
from axlearn_b200.common.config import InstantiableConfig
from axlearn_b200.common.encoder import Encoder, bert_embedding_config, bert_transformer_config
from axlearn_b200.common.layers import set_dropout_rate_recursively
from axlearn_b200.common.poolings import FirstNTokenPooling
from axlearn_b200.common.text_encoder import TextEmbeddingEncoder


def set_distilbert_config(*, vocab_size: int = 30522, num_layers: int = 6, model_dim: int = 768,
                          num_heads: int = 12, max_seq_len: int = 512, dropout_rate: float = 0.1,
                          pad_token_id: int = 0, pooler_config: Optional[InstantiableConfig] = None,
                          feed_forward_dim: Union[int, InstantiableConfig, None] = None,
                          feed_forward_act: str = "nn.gelu", layer_norm_eps: float = 1e-12,
                          remat: bool = False) -> InstantiableConfig:
    base = (RepeatedTransformerLayer if remat else StackedTransformerLayer).default_config()
    transformer = bert_transformer_config(base_cfg=base, num_layers=num_layers, num_heads=num_heads,
                                          layer_norm_epsilon=layer_norm_eps)
    transformer.layer.feed_forward.activation = feed_forward_act
    transformer.layer.feed_forward.hidden_dim = feed_forward_dim if feed_forward_dim is not None else scaled_hidden_dim(4)
    encoder = Encoder.default_config().set(
        vocab_size=vocab_size, transformer=transformer,
        emb=bert_embedding_config(max_position_embeddings=max_seq_len, layer_norm_epsilon=layer_norm_eps))
    cfg = TextEmbeddingEncoder.default_config().set(
        output_dim=model_dim, pad_token_id=pad_token_id, encoder=encoder,
        pooler=pooler_config or FirstNTokenPooling.default_config())
    set_dropout_rate_recursively(cfg, dropout_rate)
    return cfg
