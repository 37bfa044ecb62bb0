"""Contrastive image-text dual encoder (CLIP style).

Parity targets in the reference: axlearn/vision/clip.py (``CLIPTextStreamEncoder`` :60,
``CLIPImageStreamEncoder`` :190, ``CLIPFusionNetwork`` :290 with the learnable log temperature
clipped to ``[log 1, log 100]``, ``CLIPModel`` :380) on top of the generic multi-stream pattern of
axlearn/common/multi_stream_model.py; ``symmetric_contrastive_loss_from_logits`` in
axlearn/common/loss.py.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.param_init import constant_initializer
from axlearn_b200.parallel import collectives as coll

Tensor = torch.Tensor


def symmetric_contrastive_loss_from_logits(logits: Tensor) -> Tensor:
    """``logits [N, N]`` with matching pairs on the diagonal: mean of the two cross entropies."""
    target = torch.arange(logits.shape[0], device=logits.device)
    return 0.5 * (F.cross_entropy(logits.float(), target) + F.cross_entropy(logits.float().t(), target))


class StreamEncoder(BaseLayer):
    """Wraps an encoder whose ``predict(input_batch)`` returns ``{"pooled": [B, D]}`` (ViT) or
    whose call returns ``[B, T, D]`` token states (text encoder; pooled at the last live token or
    by mean) and projects to the shared embedding space, L2-normalised."""

    @config_class
    class Config(BaseLayer.Config):
        encoder: Required[InstantiableConfig] = REQUIRED
        encoder_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        input_key: Required[str] = REQUIRED          # "image" or "text"
        projection: InstantiableConfig = Linear.default_config().set(bias=False)
        pad_token_id: int = 0

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", cfg.encoder)
        self._add_child("projection", cfg.projection.clone(input_dim=cfg.encoder_dim, output_dim=cfg.output_dim))

    def forward(self, input_batch: dict) -> Tensor:
        cfg = self._config
        data = input_batch[cfg.input_key]
        if cfg.input_key == "image":
            pooled = self.encoder.predict({"image": data})["pooled"]
        else:
            states = self.encoder(data)
            states = states["hidden_states"] if isinstance(states, dict) else states
            live = (data != cfg.pad_token_id)
            last = (live.long().sum(dim=1) - 1).clamp_min(0)
            pooled = states[torch.arange(states.shape[0], device=states.device), last]
        return F.normalize(self.projection(pooled).float(), dim=-1)


class CLIPModel(BaseModel):
    @config_class
    class Config(BaseModel.Config):
        image_stream: Required[InstantiableConfig] = REQUIRED
        text_stream: Required[InstantiableConfig] = REQUIRED
        log_logit_scale_init: float = math.log(1 / 0.07)
        # Gather embeddings over the data-parallel ranks so that every rank contrasts against the
        # global batch (gradients flow back to the local rows only).
        gather_across_ranks: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("image_stream", cfg.image_stream)
        self._add_child("text_stream", cfg.text_stream)

    def _create_layer_parameter_specs(self):
        return {"log_logit_scale": ParameterSpec(
            shape=(1,), mesh_axes=(None,), initializer=constant_initializer(self._config.log_logit_scale_init),
            weight_decay_scale=0)}

    def predict(self, input_batch: dict) -> dict:
        return {"image_embedding": self.image_stream(input_batch), "text_embedding": self.text_stream(input_batch)}

    def forward(self, input_batch: dict):
        out = self.predict(input_batch)
        img, txt = out["image_embedding"], out["text_embedding"]
        scale = torch.exp(self.parameters["log_logit_scale"].float().clamp(0.0, math.log(100.0)))
        if self._config.gather_across_ranks and coll.axis_size(("data", "expert", "fsdp")) > 1:
            all_img = coll.all_gather(img, ("data", "expert", "fsdp"), dim=0)
            all_txt = coll.all_gather(txt, ("data", "expert", "fsdp"), dim=0)
            r = coll.axis_index(("data", "expert", "fsdp"))
            target = torch.arange(img.shape[0], device=img.device) + r * img.shape[0]
            loss = 0.5 * (F.cross_entropy(scale * img @ all_txt.t(), target) +
                          F.cross_entropy(scale * txt @ all_img.t(), target))
        else:
            logits = scale * img @ txt.t()
            loss = symmetric_contrastive_loss_from_logits(logits)
            self.add_summary("i2t_accuracy", (logits.argmax(dim=1) == torch.arange(len(img), device=img.device)).float().mean())
        self.add_summary("loss", loss.detach())
        self.add_summary("logit_scale", scale.detach())
        return loss, out
