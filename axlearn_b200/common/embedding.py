"""Embedding modules that combine token, type and position lookups.

Parity targets in the reference (axlearn/common/embedding.py): ``BaseEmbedding`` (:18),
``TransformerTextEmbeddings`` (:88), ``ModalityEmbedding``-style composition (:214).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Dropout, Embedding

Tensor = torch.Tensor


class BaseEmbedding(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED

    def forward(self, input_batch: dict) -> Tensor:
        raise NotImplementedError(type(self))

    def attend(self, x: Tensor) -> Tensor:
        raise NotImplementedError(type(self))


class LearnedPositionalEmbedding(BaseLayer):
    """Learned absolute positions: weight ``[1, max_len, dim]``."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        shape: Required[tuple] = REQUIRED  # (max_len,)

    def _create_layer_parameter_specs(self):
        from axlearn_b200.common.base_layer import ParameterSpec
        from axlearn_b200.common.param_init import FanAxes

        cfg = self._config
        return {
            "weight": ParameterSpec(
                shape=(1,) + tuple(cfg.shape) + (cfg.dim,),
                mesh_axes=(None,) * (len(cfg.shape) + 2),
                fan_axes=FanAxes(in_axis=-2, out_axis=-1, batch_axis=0),
            )
        }

    def forward(self, positions: Tensor) -> Tensor:
        w = self.parameters["weight"][0]
        return w[positions.long()]


class TransformerTextEmbeddings(BaseEmbedding):
    """token_emb (+ type_emb) (+ pos_emb) -> [norm] -> dropout."""

    @config_class
    class Config(BaseEmbedding.Config):
        vocab_size: Required[int] = REQUIRED
        token_emb: InstantiableConfig = Embedding.default_config()
        type_emb: Optional[InstantiableConfig] = None
        pos_emb: Optional[InstantiableConfig] = None
        norm: Optional[InstantiableConfig] = None
        dropout: InstantiableConfig = Dropout.default_config()
        soft_cap_logits: Optional[float] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("token_emb", cfg.token_emb.clone(dim=cfg.dim, num_embeddings=cfg.vocab_size))
        if cfg.type_emb is not None:
            self._add_child("type_emb", cfg.type_emb.clone(dim=cfg.dim))
        if cfg.pos_emb is not None:
            self._add_child("pos_emb", cfg.pos_emb.clone(dim=cfg.dim))
        if cfg.norm is not None:
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.dim))
        self._add_child("dropout", cfg.dropout)

    def forward(self, input_batch: dict) -> Tensor:
        inputs = input_batch["inputs"]
        x = self.token_emb(inputs)
        if "type_emb" in self._children:
            token_type_ids = input_batch.get("token_type_ids")
            if token_type_ids is None:          # every token is of type 0, as in the reference
                token_type_ids = torch.zeros_like(inputs)
            x = x + self.type_emb(token_type_ids)
        if "pos_emb" in self._children:
            positions = input_batch.get("positions")
            if positions is None:
                positions = torch.arange(inputs.shape[1], device=inputs.device)[None]
            x = x + self.pos_emb(positions)
        if "norm" in self._children:
            x = self.norm(x)
        return self.dropout(x)

    def attend(self, x: Tensor) -> Tensor:
        logits = self.token_emb.attend(x)
        cap = self._config.soft_cap_logits
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits


class SinusoidalPositionalEmbedding(BaseLayer):
    """Fixed sinusoidal position embeddings (reference: axlearn/common/layers.py
    ``SinusoidalPositionalEmbedding``): ``[sin(p / s_i) | cos(p / s_i)]`` with timescales ``s_i``
    spaced geometrically between ``min_timescale`` and ``max_timescale``."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        min_timescale: float = 1.0
        max_timescale: float = 10000.0

    def forward(self, positions: torch.Tensor) -> torch.Tensor:
        """``positions [...]`` -> ``[..., dim]``."""
        import math

        cfg = self._config
        half = cfg.dim // 2
        log_inc = math.log(cfg.max_timescale / cfg.min_timescale) / max(1, half - 1)
        inv = cfg.min_timescale * torch.exp(-log_inc * torch.arange(half, device=positions.device, dtype=torch.float32))
        scaled = positions.float()[..., None] * inv
        emb = torch.cat([torch.sin(scaled), torch.cos(scaled)], dim=-1)
        if cfg.dim % 2:
            emb = torch.nn.functional.pad(emb, (0, 1))
        return emb
