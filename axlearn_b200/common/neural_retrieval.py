"""Dense passage retrieval (DPR) configurations: BERT towers and an in-batch contrastive loss.

Reference: axlearn/common/neural_retrieval.py (:28 ``set_bert_dpr_encoder_config``, :75
``set_dpr_model_config``, :106 ``set_siamese_dpr_model_config``).
"""

from __future__ import annotations

from typing import Optional

from axlearn_b200.common.config import InstantiableConfig
from axlearn_b200.common.encoder import Encoder, bert_embedding_config, bert_transformer_config
from axlearn_b200.common.layers import RedirectToSharedModule
from axlearn_b200.common.param_init import DefaultInitializer, WeightInitializer
from axlearn_b200.common.text_dual_encoder import (
    TEXT_DUAL_ENCODER_SHARED_MODULE_NAME,
    TextEmbeddingAsymmetricContrastiveLossLayer,
    TextEmbeddingDualEncoder,
    TextEmbeddingStreamEncoder,
)
from axlearn_b200.common.text_encoder import TextEmbeddingEncoder

QUERY_ENCODER_NAME = "query_encoder"
PASSAGE_ENCODER_NAME = "passage_encoder"


def hf_param_init() -> InstantiableConfig:
    """Normal(0, 0.02) weights, the Hugging Face BERT initialisation."""
    return DefaultInitializer.default_config().set(init_by_param_name={
        ".*weight$": WeightInitializer.default_config().set(fan=None, scale=0.02, distribution="normal")})


def set_bert_dpr_encoder_config(*, vocab_size: int, num_layers: int, model_dim: int, num_heads: int,
                                max_seq_len: int = 512, pad_token_id: int = 0,
                                feed_forward_act: str = "exact_gelu",
                                output_norm: Optional[InstantiableConfig] = None,
                                remat: bool = False) -> InstantiableConfig:
    """A BERT tower whose first-token state is the embedding (no projection)."""
    base = None
    if remat:
        from axlearn_b200.common.attention import RepeatedTransformerLayer
        base = RepeatedTransformerLayer.default_config()
    transformer = bert_transformer_config(num_layers=num_layers, num_heads=num_heads, base_cfg=base)
    transformer.layer.feed_forward.activation = feed_forward_act
    emb = bert_embedding_config(max_position_embeddings=max_seq_len, type_vocab_size=2)
    for part in ("token_emb", "pos_emb", "type_emb"):
        getattr(emb, part).param_init = hf_param_init()
    encoder = Encoder.default_config().set(vocab_size=vocab_size, emb=emb, transformer=transformer)
    text = TextEmbeddingEncoder.default_config().set(pad_token_id=pad_token_id, encoder=encoder)
    return TextEmbeddingStreamEncoder.default_config().set(
        output_dim=model_dim, hidden_dim=model_dim, text_encoder=text, output_proj=None, output_norm=output_norm)


def _contrastive(scale: float) -> InstantiableConfig:
    return TextEmbeddingAsymmetricContrastiveLossLayer.default_config().set(
        left_encoder_name=QUERY_ENCODER_NAME, right_encoder_name=PASSAGE_ENCODER_NAME,
        contrastive_loss_scale_factor=scale)


def set_dpr_model_config(*, query_encoder_cfg: InstantiableConfig, passage_encoder_cfg: InstantiableConfig,
                         contrastive_loss_scale_factor: float = 1.0) -> InstantiableConfig:
    """Two separate towers."""
    return TextEmbeddingDualEncoder.default_config().set(
        param_init=hf_param_init(),
        stream_encoder={QUERY_ENCODER_NAME: query_encoder_cfg, PASSAGE_ENCODER_NAME: passage_encoder_cfg},
        fusion_network={"contrastive_fusion_network": _contrastive(contrastive_loss_scale_factor)})


def set_siamese_dpr_model_config(*, shared_encoder_cfg: InstantiableConfig,
                                 contrastive_loss_scale_factor: float = 1.0) -> InstantiableConfig:
    """One tower used for queries and passages."""
    passage = RedirectToSharedModule.default_config().set(shared_module=TEXT_DUAL_ENCODER_SHARED_MODULE_NAME)
    return TextEmbeddingDualEncoder.default_config().set(
        param_init=hf_param_init(),
        stream_encoder={QUERY_ENCODER_NAME: shared_encoder_cfg, PASSAGE_ENCODER_NAME: passage},
        fusion_network={"contrastive_fusion_network": _contrastive(contrastive_loss_scale_factor)},
        shared_encoder_name=QUERY_ENCODER_NAME)
