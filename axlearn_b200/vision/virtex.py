"""VirTex: learning visual representations from captions with a bidirectional captioning objective.

Counterpart of axlearn/vision/virtex.py (``VirTexModel``: visual backbone, a projection of its
feature map, and forward / backward transformer captioning decoders).  The image's feature map is
projected to the decoder width and flattened into tokens; one decoder predicts the caption left to
right, the other right to left (the caption is reversed inside its live length); the loss is the
sum of the two next-token cross-entropies.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from axlearn_b200.common.attention import TransformerAttentionLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.embedding import LearnedPositionalEmbedding
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.metrics import WeightedSummary

Tensor = torch.Tensor


def reverse_within_length(ids: Tensor, pad_id: int) -> Tensor:
    """Reverses every row's live prefix and leaves its padding at the end."""
    live = ids != pad_id
    n = live.sum(dim=1, keepdim=True)
    pos = torch.arange(ids.shape[1], device=ids.device)[None]
    src = torch.where(pos < n, n - 1 - pos, pos)
    return torch.gather(ids, 1, src)


def caption_decoder_config(*, vocab_size: int, dim: int, num_layers: int, num_heads: int, max_len: int = 32) -> InstantiableConfig:
    cfg = Decoder.default_config().set(vocab_size=vocab_size, dim=dim)
    cfg.emb.pos_emb = LearnedPositionalEmbedding.default_config().set(shape=(max_len,))
    cfg.transformer.num_layers = num_layers
    layer = cfg.transformer.layer
    layer.self_attention.attention.set(num_heads=num_heads, causal=True)
    layer.cross_attention = TransformerAttentionLayer.default_config().set(source_dim=dim)
    layer.cross_attention.attention.num_heads = num_heads
    layer.feed_forward.hidden_dim = 4 * dim
    return cfg


class VirTexModel(BaseModel):
    """``input_batch = {"image": [B, H, W, 3], "caption_tokens": [B, T]}`` where a caption is
    ``BOS w1 ... wn EOS`` followed by padding."""

    @config_class
    class Config(BaseModel.Config):
        visual: Required[InstantiableConfig] = REQUIRED            # backbone returning endpoints
        visual_feature: str = "5"                                  # which endpoint feeds the decoders
        textual_dim: Required[int] = REQUIRED
        forward_decoder: Required[InstantiableConfig] = REQUIRED
        backward_decoder: Required[InstantiableConfig] = REQUIRED
        bidirectional: bool = True
        pad_token_id: int = 0

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("visual", cfg.visual)
        self._add_child("visual_projection", Linear.default_config().set(
            input_dim=self.visual.endpoints_dims[cfg.visual_feature], output_dim=cfg.textual_dim, bias=True))
        self._add_child("forward_decoder", cfg.forward_decoder.clone(pad_token_id=cfg.pad_token_id))
        if cfg.bidirectional:
            self._add_child("backward_decoder", cfg.backward_decoder.clone(pad_token_id=cfg.pad_token_id))

    def embed_image(self, image: Tensor) -> Tensor:
        """``[B, H, W, 3] -> [B, h * w, textual_dim]`` visual tokens."""
        feat = self.visual(image)[self._config.visual_feature]
        return self.visual_projection(feat.reshape(feat.shape[0], -1, feat.shape[-1]))

    def _caption_loss(self, decoder, tokens: Tensor, visual_tokens: Tensor):
        pad = self._config.pad_token_id
        out = decoder(input_batch={"input_ids": tokens[:, :-1]}, cross_attention_data=visual_tokens)
        logits = decoder.compute_logits(out).float()
        labels = tokens[:, 1:]
        live = labels != pad
        per = F.cross_entropy(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="none").reshape(labels.shape)
        n = live.sum().clamp_min(1)
        return (per * live).sum() / n, n, logits

    def predict(self, input_batch: dict) -> dict:
        return {"visual_tokens": self.embed_image(input_batch["image"])}

    def forward(self, input_batch: dict):
        cfg = self._config
        visual_tokens = self.embed_image(input_batch["image"])
        tokens = input_batch["caption_tokens"]
        fwd, n, logits = self._caption_loss(self.forward_decoder, tokens, visual_tokens)
        self.add_summary("loss/forward", WeightedSummary(fwd.detach(), n))
        loss = fwd
        if cfg.bidirectional:
            bwd, n_b, _ = self._caption_loss(self.backward_decoder, reverse_within_length(tokens, cfg.pad_token_id), visual_tokens)
            self.add_summary("loss/backward", WeightedSummary(bwd.detach(), n_b))
            loss = loss + bwd
        return loss, {"visual_tokens": visual_tokens, "forward_logits": logits}
