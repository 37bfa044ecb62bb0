"""Transformer encoders and encoder-only / encoder-decoder models.

Parity targets in the reference: ``Encoder`` / ``CausalEncoder`` (axlearn/common/encoder.py:
``emb -> transformer -> [output norm] -> [pooler]`` over padded ``input_ids`` with bidirectional
attention, segment ids and token types), ``BertModel`` with MLM head, pooler and sequence
classification head (axlearn/common/bert.py), ``EncoderDecoderModel`` with teacher-forced
cross-entropy (axlearn/common/encoder_decoder.py; T5-style when configured with relative
position biases) and ``VisionTransformer`` (axlearn/vision or common/vision_transformer.py:
convolutional patch embedding, class token or pooling, classification head).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200 import ops
from axlearn_b200.common.attention import StackedTransformerLayer, TransformerLayer
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.embedding import LearnedPositionalEmbedding, TransformerTextEmbeddings
from axlearn_b200.common.layers import Dropout, LayerNorm, Linear, get_activation_fn
from axlearn_b200.common.param_init import gaussian_initializer
from axlearn_b200.common.poolings import AveragePooling, FirstNTokenPooling

Tensor = torch.Tensor
NEG_INF = -1e9


def _padding_bias(live: Tensor, dtype) -> Tensor:
    """``[B, 1, 1, S]`` additive bias that hides padding keys."""
    return torch.where(live[:, None, None, :], 0.0, NEG_INF).to(dtype)


class Encoder(BaseLayer):
    """Bidirectional transformer over ``input_ids [B, T]`` (padding = ``pad_token_id``)."""

    @config_class
    class Config(BaseLayer.Config):
        vocab_size: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        pad_token_id: int = 0
        emb: InstantiableConfig = TransformerTextEmbeddings.default_config()
        transformer: InstantiableConfig = StackedTransformerLayer.default_config()
        output: Optional[InstantiableConfig] = None      # e.g. a final LayerNorm
        output_dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("emb", cfg.emb.clone(dim=cfg.dim, vocab_size=cfg.vocab_size))
        self._add_child("transformer", cfg.transformer.clone(input_dim=cfg.dim))
        if cfg.output is not None:
            self._add_child("output", cfg.output.clone(input_dim=cfg.dim))
        self._add_child("output_dropout", cfg.output_dropout)

    def forward(self, input_ids: Tensor, *, input_segment_ids: Optional[Tensor] = None,
                token_type_ids: Optional[Tensor] = None, positions: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        live = input_ids != cfg.pad_token_id
        x = self.emb({"inputs": input_ids, "token_type_ids": token_type_ids, "positions": positions})
        bias = _padding_bias(live, x.dtype)
        if input_segment_ids is not None:
            same = input_segment_ids[:, :, None] == input_segment_ids[:, None, :]
            bias = bias + torch.where(same[:, None], 0.0, NEG_INF).to(x.dtype)
        x = self.transformer(x, self_attention_logit_biases=bias).data
        if "output" in self._children:
            x = self.output(x)
        return self.output_dropout(x)

    def attend(self, x: Tensor) -> Tensor:
        return self.emb.attend(x)


class CausalEncoder(Encoder):
    """An encoder with causal self-attention (e.g. the text tower of contrastive models)."""

    def forward(self, input_ids, **kwargs):
        cfg = self._config
        live = input_ids != cfg.pad_token_id
        x = self.emb({"inputs": input_ids, "token_type_ids": kwargs.get("token_type_ids"),
                      "positions": kwargs.get("positions")})
        t = input_ids.shape[1]
        causal = torch.tril(torch.ones(t, t, dtype=torch.bool, device=input_ids.device))
        bias = _padding_bias(live, x.dtype) + torch.where(causal[None, None], 0.0, NEG_INF).to(x.dtype)
        x = self.transformer(x, self_attention_logit_biases=bias).data
        if "output" in self._children:
            x = self.output(x)
        return self.output_dropout(x)


# ------------------------------------------------------------------------------------------
# BERT.
# ------------------------------------------------------------------------------------------


class BertLMHead(BaseLayer):
    """transform (dense + activation + norm) then logits through the tied token embedding plus
    an output bias."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        vocab_size: Required[int] = REQUIRED
        activation: str = "nn.gelu"
        norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("transform", Linear.default_config().set(input_dim=cfg.input_dim, output_dim=cfg.input_dim))
        self._add_child("norm", cfg.norm.clone(input_dim=cfg.input_dim))

    def _create_layer_parameter_specs(self):
        return {"output_bias": ParameterSpec(shape=(self._config.vocab_size,), mesh_axes=(None,),
                                             initializer=gaussian_initializer(0.0))}

    def forward(self, x: Tensor, *, attend) -> Tensor:
        h = self.norm(get_activation_fn(self._config.activation)(self.transform(x)))
        return attend(h) + self.parameters["output_bias"].to(h.dtype)


class BertModel(BaseModel):
    """Masked-LM pre-training model: ``forward`` takes ``input_ids`` (with ``[MASK]`` already
    applied), ``target_labels`` (``ignore_target_label`` where not masked) and returns the MLM
    loss; ``predict`` also returns the pooled ``[CLS]`` representation."""

    @config_class
    class Config(BaseModel.Config):
        vocab_size: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        encoder: InstantiableConfig = Encoder.default_config()
        head: InstantiableConfig = BertLMHead.default_config()
        ignore_target_label: int = 0
        num_classes: Optional[int] = None    # adds a sequence-classification head on the pooled output

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", cfg.encoder.clone(dim=cfg.dim, vocab_size=cfg.vocab_size))
        self._add_child("head", cfg.head.clone(input_dim=cfg.dim, vocab_size=cfg.vocab_size))
        self._add_child("pooler", Linear.default_config().set(input_dim=cfg.dim, output_dim=cfg.dim))
        if cfg.num_classes:
            self._add_child("classifier", Linear.default_config().set(input_dim=cfg.dim, output_dim=cfg.num_classes))

    def predict(self, input_batch: dict) -> dict:
        x = self.encoder(input_batch["input_ids"], token_type_ids=input_batch.get("token_type_ids"))
        pooled = torch.tanh(self.pooler(x[:, 0]))
        out = {"sequence_output": x, "pooled_output": pooled,
               "logits": self.head(x, attend=self.encoder.attend)}
        if "classifier" in self._children:
            out["class_logits"] = self.classifier(pooled)
        return out

    def forward(self, input_batch: dict, return_aux: bool = False):
        cfg = self._config
        out = self.predict(input_batch)
        labels = input_batch["target_labels"]
        live = labels != cfg.ignore_target_label
        loss, aux = ops.reference.cross_entropy(out["logits"], labels, live_targets=live)
        self.add_summary("mlm_loss", loss.detach())
        self.add_summary("mlm_accuracy", aux["accuracy"].detach())
        if "class_logits" in out and "class_labels" in input_batch:
            cls_loss, _ = ops.reference.cross_entropy(out["class_logits"][:, None], input_batch["class_labels"][:, None])
            self.add_summary("class_loss", cls_loss.detach())
            loss = loss + cls_loss
        return loss, ({**out, **aux} if return_aux else {})


# ------------------------------------------------------------------------------------------
# Encoder-decoder.
# ------------------------------------------------------------------------------------------


class EncoderDecoderModel(BaseModel):
    """Seq2seq: ``source.input_ids`` -> encoder; ``target.input_ids`` -> decoder with
    cross-attention to the encoder output; loss = cross-entropy on ``target_labels``."""

    @config_class
    class Config(BaseModel.Config):
        encoder: Required[InstantiableConfig] = REQUIRED
        decoder: Required[InstantiableConfig] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", cfg.encoder)
        self._add_child("decoder", cfg.decoder)

    def predict(self, input_batch: dict) -> dict:
        src = input_batch["source"]["input_ids"]
        enc = self.encoder(src)
        live = src != self.encoder.config.pad_token_id
        tgt = input_batch["target"]["input_ids"]
        cross_bias = _padding_bias(live, enc.dtype).expand(-1, -1, tgt.shape[1], -1)
        dec = self.decoder({"input_ids": tgt}, cross_attention_data=enc, cross_attention_logit_biases=cross_bias)
        return {"encoder_output": enc, **dec, "logits": self.decoder.compute_logits(dec)}

    def forward(self, input_batch: dict, return_aux: bool = False):
        out = self.predict(input_batch)
        labels = input_batch["target_labels"]
        live = labels != self.decoder.config.pad_token_id
        loss, aux = ops.reference.cross_entropy(out["logits"], labels, live_targets=live)
        self.add_summary("loss", loss.detach())
        return loss, ({**out, **aux} if return_aux else {})


def encoder_decoder_config(*, vocab_size: int, dim: int, num_layers: int, num_heads: int, max_len: int = 512):
    """A small learned-position encoder-decoder (both stacks ``num_layers`` deep)."""
    from axlearn_b200.common.attention import TransformerAttentionLayer

    def stack(cross: bool):
        layer = TransformerLayer.default_config()
        layer.self_attention.attention.num_heads = num_heads
        layer.feed_forward.hidden_dim = 4 * dim
        if cross:
            layer.cross_attention = TransformerAttentionLayer.default_config()
            layer.cross_attention.attention.num_heads = num_heads
            layer.cross_attention.source_dim = dim
        return StackedTransformerLayer.default_config().set(num_layers=num_layers, layer=layer)

    emb = lambda: TransformerTextEmbeddings.default_config().set(
        pos_emb=LearnedPositionalEmbedding.default_config().set(shape=(max_len,)))
    dec_stack = stack(True)
    dec_stack.layer.self_attention.attention.causal = True
    return EncoderDecoderModel.default_config().set(
        encoder=Encoder.default_config().set(vocab_size=vocab_size, dim=dim, emb=emb(), transformer=stack(False),
                                             output=LayerNorm.default_config()),
        decoder=Decoder.default_config().set(vocab_size=vocab_size, dim=dim, emb=emb(), transformer=dec_stack))


# ------------------------------------------------------------------------------------------
# Vision transformer.
# ------------------------------------------------------------------------------------------


class VisionTransformer(BaseModel):
    """ViT image classifier: conv patch embedding -> (+ class token, learned positions) ->
    transformer -> norm -> pooling -> linear head.  Images are ``[B, H, W, C]``."""

    @config_class
    class Config(BaseModel.Config):
        image_size: tuple = (224, 224)
        patch_size: tuple = (16, 16)
        num_channels: int = 3
        dim: Required[int] = REQUIRED
        num_classes: Required[int] = REQUIRED
        transformer: InstantiableConfig = StackedTransformerLayer.default_config()
        use_class_token: bool = True
        output_norm: InstantiableConfig = LayerNorm.default_config()
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("patch_emb", Conv2D.default_config().set(
            window=cfg.patch_size, strides=cfg.patch_size, input_dim=cfg.num_channels, output_dim=cfg.dim))
        self._num_patches = (cfg.image_size[0] // cfg.patch_size[0]) * (cfg.image_size[1] // cfg.patch_size[1])
        self._add_child("pos_emb", LearnedPositionalEmbedding.default_config().set(
            dim=cfg.dim, shape=(self._num_patches + int(cfg.use_class_token),)))
        self._add_child("transformer", cfg.transformer.clone(input_dim=cfg.dim))
        self._add_child("output_norm", cfg.output_norm.clone(input_dim=cfg.dim))
        pool = FirstNTokenPooling if cfg.use_class_token else AveragePooling
        self._add_child("pooler", pool.default_config().set(input_dim=cfg.dim, output_dim=cfg.dim))
        self._add_child("classifier", Linear.default_config().set(input_dim=cfg.dim, output_dim=cfg.num_classes))
        self._add_child("dropout", cfg.dropout)

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if not cfg.use_class_token:
            return {}
        return {"cls_token": ParameterSpec(shape=(1, 1, cfg.dim), mesh_axes=(None, None, None),
                                           initializer=gaussian_initializer(0.02))}

    def predict(self, input_batch: dict) -> dict:
        cfg = self._config
        image = input_batch["image"]
        x = self.patch_emb(image)
        b = x.shape[0]
        x = x.reshape(b, -1, cfg.dim)
        if cfg.use_class_token:
            x = torch.cat([self.parameters["cls_token"].to(x.dtype).expand(b, -1, -1), x], dim=1)
        x = x + self.pos_emb(torch.arange(x.shape[1], device=x.device)[None])
        x = self.output_norm(self.transformer(self.dropout(x)).data)
        pooled = self.pooler(x)[:, 0]
        return {"encoded": x, "pooled": pooled, "logits": self.classifier(pooled)}

    def forward(self, input_batch: dict, return_aux: bool = False):
        out = self.predict(input_batch)
        labels = input_batch["label"]
        loss, aux = ops.reference.cross_entropy(out["logits"][:, None], labels[:, None])
        self.add_summary("loss", loss.detach())
        self.add_summary("accuracy", aux["accuracy"].detach())
        return loss, ({**out, **aux} if return_aux else {})
