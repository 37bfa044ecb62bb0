"""One embedding vector (or a few) per token sequence: a transformer encoder plus a pooler.

Reference: axlearn/common/text_encoder.py:20-69 (``TextEmbeddingEncoder``).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.encoder import Encoder
from axlearn_b200.common.poolings import FirstNTokenPooling

ENCODED_HIDDEN_STATES = "encoded_hidden_states"
TEXT_EMBEDDINGS = "text_embeddings"


class TextEmbeddingEncoder(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        output_dim: Required[int] = REQUIRED
        hidden_dim: Optional[int] = None            # encoder width; default output_dim
        pad_token_id: Required[int] = REQUIRED
        encoder: InstantiableConfig = Encoder.default_config()
        pooler: InstantiableConfig = FirstNTokenPooling.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        hidden = cfg.hidden_dim or cfg.output_dim
        self._add_child("encoder", cfg.encoder.clone(dim=hidden, pad_token_id=cfg.pad_token_id))
        self._add_child("pooler", cfg.pooler.clone(input_dim=hidden, output_dim=cfg.output_dim))

    def forward(self, input_ids: torch.Tensor) -> dict:
        """``input_ids [batch, length]`` -> hidden states ``[batch, length, hidden]`` and
        embeddings ``[batch, num_outputs, output_dim]``."""
        x = self.encoder(input_ids)
        paddings = input_ids == self._config.pad_token_id
        return {ENCODED_HIDDEN_STATES: x, TEXT_EMBEDDINGS: self.pooler(x, paddings=paddings)}
