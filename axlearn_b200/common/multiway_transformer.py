"""Multiway transformers (VLMo / BEiT-3): shared self-attention, one feed-forward expert per modality.

Reference: axlearn/common/multiway_transformer.py (``MultiwayTransformerLayer`` :51-240,
``MultiModalEncoder`` :243-420).  Text goes to expert 0, images to expert 1; an image-text sequence
goes to a third, fused expert when the layer has one, and is otherwise split at ``max_text_len``
between the two single-modality experts.
"""

from __future__ import annotations

from typing import Optional, Union

import torch

from axlearn_b200.common.attention import TransformerAttentionLayer, TransformerFeedForwardLayer, scaled_hidden_dim
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.embedding import LearnedPositionalEmbedding, TransformerTextEmbeddings
from axlearn_b200.common.layers import Dropout, Embedding, LayerNorm
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.common.poolings import FirstNTokenPooling

Tensor = torch.Tensor
TEXT_MODALITY, IMAGE_MODALITY, TEXT_IMAGE_MODALITY = 0, 1, 2


class MultiwayTransformerLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        self_attention: InstantiableConfig = TransformerAttentionLayer.default_config()
        feed_forward: InstantiableConfig = TransformerFeedForwardLayer.default_config()
        num_ffn: int = 1
        max_text_len: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("self_attention", cfg.self_attention.clone(target_dim=cfg.input_dim, source_dim=cfg.input_dim))
        for i in range(cfg.num_ffn):
            self._add_child(f"feed_forward{i}", cfg.feed_forward.clone(input_dim=cfg.input_dim))

    def forward(self, data: Tensor, *, feed_forward_index: int = 0,
                self_attention_logit_biases: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        x = self.self_attention(target=data, attention_logit_biases=self_attention_logit_biases).data
        if feed_forward_index < cfg.num_ffn:
            return getattr(self, f"feed_forward{feed_forward_index}")(x)
        if not isinstance(cfg.max_text_len, int):
            raise ValueError("routing a fused sequence without a fused expert needs max_text_len")
        text, image = x[:, :cfg.max_text_len], x[:, cfg.max_text_len:]
        return torch.cat([getattr(self, f"feed_forward{TEXT_MODALITY}")(text),
                          getattr(self, f"feed_forward{IMAGE_MODALITY}")(image)], dim=1)


class MultiModalEncoder(BaseLayer):
    """``inputs``: ``{0: token ids [B, T]}``, ``{1: images [B, H, W, C]}`` and / or
    ``{2: {0: ids, 1: images}}``; returns one pooled embedding ``[B, num_outputs, dim]`` per key."""

    @config_class
    class Config(BaseLayer.Config):
        output_dim: Required[int] = REQUIRED
        vocab_size: Required[int] = REQUIRED
        num_layers: Required[int] = REQUIRED
        image_size: tuple = (224, 224)
        patch_size: tuple = (16, 16)
        num_cls_tokens: int = 1
        use_mask_tokens: bool = False
        max_text_len: int = 64
        pad_token_id: int = 0
        layer: InstantiableConfig = MultiwayTransformerLayer.default_config().set(num_ffn=2)
        input_dropout: InstantiableConfig = Dropout.default_config()
        output_norm: InstantiableConfig = LayerNorm.default_config().set(eps=1e-6)
        pooler: InstantiableConfig = FirstNTokenPooling.default_config()

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.layer.feed_forward.set(activation="nn.gelu", hidden_dim=scaled_hidden_dim(4))
        cfg.layer.feed_forward.norm = LayerNorm.default_config().set(eps=1e-6)
        cfg.layer.self_attention.norm = LayerNorm.default_config().set(eps=1e-6)
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        d = cfg.output_dim
        self._add_child("visual_embed", Conv2D.default_config().set(
            window=cfg.patch_size, strides=cfg.patch_size, input_dim=3, output_dim=d))
        patches = (cfg.image_size[0] // cfg.patch_size[0]) * (cfg.image_size[1] // cfg.patch_size[1])
        self._add_child("visual_pos_emb", LearnedPositionalEmbedding.default_config().set(dim=d, shape=(patches + cfg.num_cls_tokens,)))
        self._add_child("text_embed", TransformerTextEmbeddings.default_config().set(
            dim=d, vocab_size=cfg.vocab_size, pos_emb=LearnedPositionalEmbedding.default_config().set(shape=(cfg.max_text_len,))))
        self._add_child("modality_emb", Embedding.default_config().set(num_embeddings=2, dim=d, param_partition_spec=(None, None)))
        self._add_child("input_dropout", cfg.input_dropout)
        for i in range(cfg.num_layers):
            self._add_child(f"layer{i}", cfg.layer.clone(input_dim=d, max_text_len=cfg.max_text_len))
        self._add_child("output_norm", cfg.output_norm.clone(input_dim=d))
        self._add_child("pooler", cfg.pooler.clone(input_dim=d, output_dim=d))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        specs = {}
        if cfg.num_cls_tokens:
            specs["cls_token"] = ParameterSpec(shape=(1, cfg.num_cls_tokens, cfg.output_dim), mesh_axes=(None, None, None),
                                               initializer=constant_initializer(0.0))
        if cfg.use_mask_tokens:
            specs["mask_token"] = ParameterSpec(shape=(1, 1, cfg.output_dim), mesh_axes=(None, None, None),
                                                initializer=constant_initializer(0.0))
        return specs

    def get_visual_embed(self, image: Tensor, *, is_masked: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        x = self.visual_embed(image)
        x = x.reshape(x.shape[0], -1, x.shape[-1])
        if cfg.use_mask_tokens and is_masked is not None:
            x = torch.where(is_masked.bool()[..., None], self.parameters["mask_token"].to(x.dtype), x)
        if cfg.num_cls_tokens:
            x = torch.cat([self.parameters["cls_token"].to(x.dtype).expand(x.shape[0], -1, -1), x], dim=1)
        x = x + self.visual_pos_emb(torch.arange(x.shape[1], device=x.device)[None])
        return x + self.modality_emb(torch.full(x.shape[:2], IMAGE_MODALITY, device=x.device))

    def get_text_embed(self, ids: Tensor) -> Tensor:
        x = self.text_embed({"inputs": ids})
        return x + self.modality_emb(torch.full(x.shape[:2], TEXT_MODALITY, device=x.device))

    def _bias(self, live: Tensor, dtype) -> Tensor:
        return torch.where(live[:, None, None, :], 0.0, -1e9).to(dtype)

    def forward(self, inputs: dict, *, is_masked: Optional[Tensor] = None) -> dict:
        cfg = self._config
        out = {}
        for modality, data in inputs.items():
            if modality == TEXT_MODALITY:
                x = self.get_text_embed(data)
                live = data != cfg.pad_token_id
            elif modality == IMAGE_MODALITY:
                x = self.get_visual_embed(data, is_masked=is_masked)
                live = torch.ones(x.shape[:2], dtype=torch.bool, device=x.device)
            elif modality == TEXT_IMAGE_MODALITY:
                ids = data[TEXT_MODALITY]
                if ids.shape[1] != cfg.max_text_len:
                    raise ValueError(f"fused inputs need text padded to max_text_len={cfg.max_text_len}")
                xt, xi = self.get_text_embed(ids), self.get_visual_embed(data[IMAGE_MODALITY], is_masked=is_masked)
                x = torch.cat([xt, xi], dim=1)
                live = torch.cat([ids != cfg.pad_token_id, torch.ones(xi.shape[:2], dtype=torch.bool, device=x.device)], dim=1)
            else:
                raise ValueError(f"unsupported modality {modality}")
            x = self.input_dropout(x)
            bias = self._bias(live, x.dtype)
            for i in range(cfg.num_layers):
                x = getattr(self, f"layer{i}")(x, feed_forward_index=modality, self_attention_logit_biases=bias)
            x = self.output_norm(x)
            out[modality] = self.pooler(x, paddings=~live)
        return out
