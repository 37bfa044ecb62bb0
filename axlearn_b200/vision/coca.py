"""CoCa: contrastive captioner.  One image encoder, a unimodal text decoder (contrastive branch)
and a multimodal decoder that cross-attends to image tokens (captioning branch).

Reference: axlearn/vision/coca.py (``CoCaImageStreamEncoder``, ``CoCaLMTextStreamEncoder`` with the
unimodal / multimodal split, ``CoCaContrastiveFusionNetwork``, ``CoCaCaptioningFusionNetwork``,
``CoCaModel`` :1000-1147).  The image encoder's tokens pass through two attention poolers: one
query for the contrastive embedding and ``num_caption_queries`` queries that the captioning decoder
attends to.  The text side appends a ``[CLS]`` position to the unimodal decoder; its state is the
text embedding.  Loss = ``contrastive_weight * symmetric InfoNCE + caption_weight * next-token CE``.
CyCLIP's cyclic consistency terms (axlearn/vision/cyclip.py) are available as extra regularisers.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from axlearn_b200.common.attention import StackedTransformerLayer, TransformerAttentionLayer
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Embedding, LayerNorm, Linear
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.param_init import constant_initializer, gaussian_initializer
from axlearn_b200.common.poolings import AttentionPooling

Tensor = torch.Tensor
NEG_INF = -1e9


def cyclip_losses(image_emb: Tensor, text_emb: Tensor) -> tuple[Tensor, Tensor]:
    """(cross-modal, in-modal) cyclic consistency: the image-text similarity matrix should be
    symmetric, and image-image similarities should equal text-text similarities."""
    it = image_emb @ text_emb.t()
    cross = ((it - it.t()) ** 2).mean()
    inmodal = ((image_emb @ image_emb.t() - text_emb @ text_emb.t()) ** 2).mean()
    return cross, inmodal


class CoCaTextDecoder(BaseLayer):
    """Causal unimodal layers over ``tokens + [CLS]``, then multimodal layers (with
    cross-attention) over the token positions."""

    @config_class
    class Config(BaseLayer.Config):
        vocab_size: Required[int] = REQUIRED
        dim: Required[int] = REQUIRED
        max_len: int = 77
        pad_token_id: int = 0
        unimodal: InstantiableConfig = StackedTransformerLayer.default_config()
        multimodal: InstantiableConfig = StackedTransformerLayer.default_config()
        norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("token_emb", Embedding.default_config().set(num_embeddings=cfg.vocab_size, dim=cfg.dim,
                                                                    param_partition_spec=(None, None)))
        self._add_child("unimodal", cfg.unimodal.clone(input_dim=cfg.dim))
        multi = cfg.multimodal.clone(input_dim=cfg.dim)
        multi.layer.cross_attention = TransformerAttentionLayer.default_config().set(source_dim=cfg.dim)
        multi.layer.cross_attention.attention.num_heads = multi.layer.self_attention.attention.num_heads
        self._add_child("multimodal", multi)
        self._add_child("unimodal_norm", cfg.norm.clone(input_dim=cfg.dim))
        self._add_child("output_norm", cfg.norm.clone(input_dim=cfg.dim))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"pos_emb": ParameterSpec(shape=(cfg.max_len + 1, cfg.dim), mesh_axes=(None, None),
                                         initializer=gaussian_initializer(0.01)),
                "cls_token": ParameterSpec(shape=(1, 1, cfg.dim), mesh_axes=(None, None, None),
                                           initializer=gaussian_initializer(0.02))}

    @staticmethod
    def _causal_bias(live: Tensor) -> Tensor:
        t = live.shape[1]
        causal = torch.tril(torch.ones(t, t, dtype=torch.bool, device=live.device))
        ok = causal[None] & live[:, None, :]
        return torch.where(ok, 0.0, NEG_INF)[:, None]

    def forward(self, input_ids: Tensor, *, image_tokens: Tensor) -> dict:
        cfg = self._config
        b, t = input_ids.shape
        x = self.token_emb(input_ids)
        x = torch.cat([x, self.parameters["cls_token"].to(x.dtype).expand(b, -1, -1)], dim=1)
        x = x + self.parameters["pos_emb"][: t + 1].to(x.dtype)
        live = torch.cat([input_ids != cfg.pad_token_id, torch.ones(b, 1, dtype=torch.bool, device=x.device)], dim=1)
        uni = self.unimodal(x, self_attention_logit_biases=self._causal_bias(live).to(x.dtype)).data
        text_embedding = self.unimodal_norm(uni[:, -1])              # [CLS] sees every live token
        tokens = uni[:, :-1]
        multi = self.multimodal(tokens, self_attention_logit_biases=self._causal_bias(live[:, :-1]).to(x.dtype),
                                cross_attention_data=image_tokens).data
        hidden = self.output_norm(multi)
        return {"text_embedding": text_embedding, "logits": self.token_emb.attend(hidden)}


class CoCaModel(BaseModel):
    """``input_batch = {"image": [B, H, W, C], "text": [B, T]}``; captions are predicted from their
    own prefix (targets = ``text`` shifted left by one)."""

    @config_class
    class Config(BaseModel.Config):
        image_encoder: Required[InstantiableConfig] = REQUIRED      # predict() -> {"encoded": [B, N, D]}
        image_dim: Required[int] = REQUIRED
        text_decoder: Required[InstantiableConfig] = REQUIRED
        dim: Required[int] = REQUIRED
        num_caption_queries: int = 256
        pooler_heads: int = 8
        contrastive_weight: float = 1.0
        caption_weight: float = 2.0
        cyclip_cross_weight: float = 0.0
        cyclip_inmodal_weight: float = 0.0
        log_logit_scale_init: float = math.log(1 / 0.07)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("image_encoder", cfg.image_encoder)
        pool = AttentionPooling.default_config().set(input_dim=cfg.image_dim, output_dim=cfg.dim, num_heads=cfg.pooler_heads)
        self._add_child("contrastive_pooler", pool.clone(num_outputs=1))
        self._add_child("caption_pooler", pool.clone(num_outputs=cfg.num_caption_queries))
        self._add_child("text_decoder", cfg.text_decoder.clone(dim=cfg.dim))

    def _create_layer_parameter_specs(self):
        return {"log_logit_scale": ParameterSpec(shape=(1,), mesh_axes=(None,), weight_decay_scale=0,
                                                 initializer=constant_initializer(self._config.log_logit_scale_init))}

    def predict(self, input_batch: dict) -> dict:
        tokens = self.image_encoder.predict({"image": input_batch["image"]})["encoded"]
        image_embedding = F.normalize(self.contrastive_pooler(tokens)[:, 0].float(), dim=-1)
        out = {"image_embedding": image_embedding}
        if "text" in input_batch:
            dec = self.text_decoder(input_batch["text"], image_tokens=self.caption_pooler(tokens))
            out["text_embedding"] = F.normalize(dec["text_embedding"].float(), dim=-1)
            out["logits"] = dec["logits"]
        return out

    def forward(self, input_batch: dict):
        cfg = self._config
        out = self.predict(input_batch)
        img, txt = out["image_embedding"], out["text_embedding"]
        scale = torch.exp(self.parameters["log_logit_scale"].float().clamp(0.0, math.log(100.0)))
        sim = scale * img @ txt.t()
        target = torch.arange(sim.shape[0], device=sim.device)
        contrastive = 0.5 * (F.cross_entropy(sim, target) + F.cross_entropy(sim.t(), target))
        text = input_batch["text"]
        labels = text[:, 1:]
        live = labels != cfg.text_decoder.pad_token_id
        logits = out["logits"][:, :-1].float()
        per = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="none").reshape(labels.shape)
        n = live.sum().clamp_min(1)
        caption = (per * live).sum() / n
        loss = cfg.contrastive_weight * contrastive + cfg.caption_weight * caption
        if cfg.cyclip_cross_weight or cfg.cyclip_inmodal_weight:
            cross, inmodal = cyclip_losses(img, txt)
            loss = loss + cfg.cyclip_cross_weight * cross + cfg.cyclip_inmodal_weight * inmodal
        self.add_summary("loss/contrastive", contrastive.detach())
        self.add_summary("loss/caption", WeightedSummary(caption.detach(), n))
        self.add_summary("logit_scale", scale.detach())
        return loss, out

    @torch.no_grad()
    def generate(self, input_batch: dict, *, bos_id: int, eos_id: int, max_len: int = 32) -> Tensor:
        """Greedy captions ``[B, max_len]`` (padding after EOS)."""
        cfg = self._config
        tokens = self.caption_pooler(self.image_encoder.predict({"image": input_batch["image"]})["encoded"])
        b = tokens.shape[0]
        pad = cfg.text_decoder.pad_token_id
        ids = torch.full((b, 1), bos_id, dtype=torch.long, device=tokens.device)
        done = torch.zeros(b, dtype=torch.bool, device=tokens.device)
        for _ in range(max_len - 1):
            logits = self.text_decoder(ids, image_tokens=tokens)["logits"][:, -1]
            nxt = torch.where(done, torch.full((b,), pad, device=ids.device), logits.argmax(-1))
            ids = torch.cat([ids, nxt[:, None]], dim=1)
            done = done | (nxt == eos_id)
            if done.all():
                break
        return F.pad(ids, (0, max_len - ids.shape[1]), value=pad)
