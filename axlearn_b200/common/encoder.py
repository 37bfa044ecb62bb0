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


class NonLinear(BaseLayer):
    """``norm(activation(linear(x)))`` (children ``linear`` and ``norm``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Optional[int] = None
        linear: InstantiableConfig = Linear.default_config()
        activation: str = "nn.gelu"
        norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        out = cfg.output_dim or cfg.input_dim
        self._add_child("linear", cfg.linear.clone(input_dim=cfg.input_dim, output_dim=out))
        self._add_child("norm", cfg.norm.clone(input_dim=out))

    def forward(self, x: Tensor) -> Tensor:
        return self.norm(get_activation_fn(self._config.activation)(self.linear(x)))


class BertLMHead(BaseLayer):
    """Masked-LM head (reference: axlearn/common/bert.py ``BertLMHead``): ``transform`` (dense +
    activation + norm), logits through the tied token embedding plus ``output_bias``; the loss
    ignores positions whose target equals ``ignored_target_id``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_classes: Required[int] = REQUIRED          # = vocabulary size
        transform: InstantiableConfig = NonLinear.default_config()
        ignored_target_id: int = 0
        # Maps hidden states to logits when the caller passes no ``attend``: an own projection, or
        # a ``RedirectToSharedModule`` onto a shared token embedding's ``attend``.
        inner_head: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("transform", cfg.transform.clone(input_dim=cfg.input_dim))
        if cfg.inner_head is not None:
            head = cfg.inner_head.clone()
            if "input_dim" in head.keys():
                head.set(input_dim=cfg.input_dim, output_dim=cfg.num_classes)
            self._add_child("inner_head", head)

    def _create_layer_parameter_specs(self):
        return {"output_bias": ParameterSpec(shape=(self._config.num_classes,), mesh_axes=(None,),
                                             initializer=gaussian_initializer(0.0))}

    def forward(self, *, sequence_output: Tensor, attend=None, **unused) -> dict:
        h = self.transform(sequence_output)
        if attend is None:
            if "inner_head" not in self._children:
                raise ValueError("BertLMHead needs `attend` or a configured `inner_head`")
            attend = self.inner_head
        return {"logits": attend(h) + self.parameters["output_bias"].to(h.dtype)}

    def loss(self, *, logits: Tensor, target_labels: Tensor):
        live = target_labels != self._config.ignored_target_id
        return ops.reference.cross_entropy(logits, target_labels, live_targets=live)


class BertPooler(BaseLayer):
    """``tanh(linear(first token))`` with dropout."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        linear: InstantiableConfig = Linear.default_config()
        dropout: InstantiableConfig = Dropout.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("linear", cfg.linear.clone(input_dim=cfg.input_dim, output_dim=cfg.input_dim))
        self._add_child("dropout", cfg.dropout)

    def forward(self, x: Tensor) -> Tensor:
        return self.dropout(torch.tanh(self.linear(x[:, 0])))


class BertSequenceClassificationHead(BaseLayer):
    """``pooler`` + ``output`` projection to ``num_classes`` (reference: axlearn/common/bert.py
    ``BertSequenceClassificationHead``); cross-entropy over ``target_labels [B]``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_classes: Required[int] = REQUIRED
        pooler: InstantiableConfig = BertPooler.default_config()
        output: InstantiableConfig = Linear.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("pooler", cfg.pooler.clone(input_dim=cfg.input_dim))
        self._add_child("output", cfg.output.clone(input_dim=cfg.input_dim, output_dim=cfg.num_classes))

    def forward(self, *, sequence_output: Tensor, **unused) -> dict:
        pooled = self.pooler(sequence_output)
        return {"pooled_output": pooled, "logits": self.output(pooled)}

    def loss(self, *, logits: Tensor, target_labels: Tensor):
        return ops.reference.cross_entropy(logits[:, None], target_labels.reshape(-1)[:, None])


class BertModel(BaseModel):
    """``encoder`` + ``head`` (reference: axlearn/common/bert.py ``BertModel``): with the default
    ``BertLMHead`` a masked-LM model (``input_ids`` with ``[MASK]`` applied, ``target_labels`` equal
    to ``ignored_target_id`` where not masked); with ``BertSequenceClassificationHead`` a sequence
    classifier.  ``predict`` returns ``sequence_output`` and the head's outputs."""

    @config_class
    class Config(BaseModel.Config):
        vocab_size: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        encoder: InstantiableConfig = Encoder.default_config()
        head: InstantiableConfig = BertLMHead.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", cfg.encoder.clone(dim=cfg.dim, vocab_size=cfg.vocab_size))
        head = cfg.head.clone(input_dim=cfg.dim)
        if head.klass is BertLMHead:
            head.num_classes = cfg.vocab_size
        self._add_child("head", head)

    def predict(self, input_batch: dict) -> dict:
        x = self.encoder(input_batch["input_ids"], token_type_ids=input_batch.get("token_type_ids"))
        return {"sequence_output": x, **self.head(sequence_output=x, attend=self.encoder.attend)}

    def forward(self, input_batch: dict, return_aux: bool = False):
        out = self.predict(input_batch)
        loss, aux = self.head.loss(logits=out["logits"], target_labels=input_batch["target_labels"])
        self.add_summary("loss", loss.detach())
        self.add_summary("accuracy", aux["accuracy"].detach())
        return loss, ({**out, **aux} if return_aux else {})


def bert_embedding_config(*, max_position_embeddings: Optional[int] = 512, layer_norm_epsilon: Optional[float] = None,
                          type_vocab_size: Optional[int] = None):
    """token + (learned position) + (token type) embeddings followed by LayerNorm."""
    from axlearn_b200.common.layers import Embedding

    norm = LayerNorm.default_config()
    if layer_norm_epsilon is not None:
        norm.eps = layer_norm_epsilon
    cfg = TransformerTextEmbeddings.default_config().set(norm=norm)
    if max_position_embeddings is not None:
        cfg.pos_emb = LearnedPositionalEmbedding.default_config().set(shape=(max_position_embeddings,))
    if type_vocab_size is not None:
        cfg.type_emb = Embedding.default_config().set(num_embeddings=type_vocab_size)
    return cfg


def bert_transformer_config(*, num_layers: int = 12, num_heads: int = 12, layer_norm_epsilon: float = 1e-12,
                            base_cfg: Optional[InstantiableConfig] = None):
    """Post-norm layers with a 4x GELU feed-forward."""
    from axlearn_b200.common.attention import scaled_hidden_dim

    base_cfg = base_cfg.clone() if base_cfg is not None else StackedTransformerLayer.default_config()
    layer_cfg = TransformerLayer.default_config()
    layer_cfg.feed_forward.set(activation="nn.gelu", hidden_dim=scaled_hidden_dim(4), structure="postnorm")
    layer_cfg.feed_forward.norm.eps = layer_norm_epsilon
    layer_cfg.self_attention.norm.eps = layer_norm_epsilon
    layer_cfg.self_attention.attention.num_heads = num_heads
    layer_cfg.self_attention.structure = "postnorm"
    return base_cfg.set(num_layers=num_layers, layer=layer_cfg)


def bert_model_config(*, vocab_size: int, hidden_dim: int = 768, num_layers: int = 12, num_heads: int = 12,
                      max_position_embeddings: int = 512, type_vocab_size: Optional[int] = 2,
                      layer_norm_epsilon: float = 1e-12, dropout_rate: float = 0.0,
                      head_cfg: Optional[InstantiableConfig] = None) -> "BertModel.Config":
    """BERT-base by default (reference: axlearn/common/bert.py ``bert_model_config``)."""
    from axlearn_b200.common.layers import set_dropout_rate_recursively

    encoder = Encoder.default_config().set(
        pad_token_id=0,
        emb=bert_embedding_config(max_position_embeddings=max_position_embeddings,
                                  layer_norm_epsilon=layer_norm_epsilon, type_vocab_size=type_vocab_size),
        transformer=bert_transformer_config(num_layers=num_layers, num_heads=num_heads,
                                            layer_norm_epsilon=layer_norm_epsilon))
    head = head_cfg or BertLMHead.default_config()
    if head.klass is BertLMHead:
        head.transform.norm.eps = layer_norm_epsilon
    cfg = BertModel.default_config().set(vocab_size=vocab_size, dim=hidden_dim, encoder=encoder, head=head)
    set_dropout_rate_recursively(cfg, dropout_rate)
    return cfg


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
