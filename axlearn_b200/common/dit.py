"""Diffusion transformer (DiT) blocks.

Parity target in the reference: axlearn/common/dit.py -- ``TimeStepEmbedding`` (:60: sinusoidal
features -> two-layer MLP), ``LabelEmbedding`` (:130: class embeddings with random drop to the
"null" class for classifier-free guidance), ``AdaptiveLayerNormModulation`` (:190: SiLU -> linear
to ``num_outputs * dim`` shift / scale / gate vectors), ``DiTFeedForwardLayer`` / ``DiTAttentionLayer``
(:250-460: LayerNorm without parameters, ``x * (1 + scale) + shift``, residual gated by ``gate``),
``DiTBlock`` (:470), ``DiTFinalLayer`` (:540: modulated norm -> linear, zero-initialised).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.attention import MultiheadAttention
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Embedding, LayerNormStateless, Linear, get_activation_fn
from axlearn_b200.common.param_init import ConstantInitializer, DefaultInitializer

Tensor = torch.Tensor


def _zero_init() -> InstantiableConfig:
    """Every parameter of the layer starts at zero (adaLN-zero)."""
    return DefaultInitializer.default_config().set(
        init_by_param_name={".*": ConstantInitializer.default_config().set(value=0.0)})


def modulate(x: Tensor, *, shift: Tensor, scale: Tensor) -> Tensor:
    """``x [B, T, D]``, ``shift / scale [B, D]`` (or ``[B, 1, D]``)."""
    if shift.dim() == 2:
        shift, scale = shift[:, None], scale[:, None]
    return x * (1 + scale) + shift


class TimeStepEmbedding(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        output_dim: Required[int] = REQUIRED
        pos_embed_dim: int = 256
        max_timescale: float = 10000.0
        activation: str = "nn.silu"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("linear1", Linear.default_config().set(input_dim=cfg.pos_embed_dim, output_dim=cfg.output_dim))
        self._add_child("linear2", Linear.default_config().set(input_dim=cfg.output_dim, output_dim=cfg.output_dim))

    def forward(self, positions: Tensor) -> Tensor:
        """``positions [B]`` (diffusion time steps, possibly fractional) -> ``[B, output_dim]``."""
        cfg = self._config
        half = cfg.pos_embed_dim // 2
        freqs = torch.exp(-math.log(cfg.max_timescale) * torch.arange(half, device=positions.device).float() / half)
        args = positions.float()[:, None] * freqs[None]
        feats = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
        return self.linear2(get_activation_fn(cfg.activation)(self.linear1(feats)))


class LabelEmbedding(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        num_classes: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        dropout_rate: float = 0.1

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        # One extra row: the "no label" class that dropped labels map to.
        self._add_child("emb", Embedding.default_config().set(num_embeddings=cfg.num_classes + 1, dim=cfg.output_dim))

    def forward(self, labels: Tensor) -> Tensor:
        cfg = self._config
        if self.is_training and cfg.dropout_rate > 0:
            drop = prng.uniform(self.prng_key, labels.shape, device=labels.device) < cfg.dropout_rate
            labels = torch.where(drop, torch.full_like(labels, cfg.num_classes), labels)
        return self.emb(labels)


class AdaptiveLayerNormModulation(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        num_outputs: Required[int] = REQUIRED
        activation: str = "nn.silu"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("linear", Linear.default_config().set(
            input_dim=cfg.dim, output_dim=cfg.num_outputs * cfg.dim, param_init=_zero_init()))

    def forward(self, condition: Tensor) -> tuple:
        x = self.linear(get_activation_fn(self._config.activation)(condition))
        return tuple(x.chunk(self._config.num_outputs, dim=-1))


class DiTBlock(BaseLayer):
    """Self-attention and feed-forward sub-layers, each ``x + gate * f(modulate(norm(x)))`` with
    the six modulation vectors computed from the conditioning embedding."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        hidden_dim_scale: float = 4.0
        attention: InstantiableConfig = MultiheadAttention.default_config()
        activation: str = "nn.gelu"
        norm_eps: float = 1e-6

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        d = cfg.input_dim
        self._add_child("adaln", AdaptiveLayerNormModulation.default_config().set(dim=d, num_outputs=6))
        self._add_child("norm1", LayerNormStateless.default_config().set(input_dim=d, eps=cfg.norm_eps))
        self._add_child("norm2", LayerNormStateless.default_config().set(input_dim=d, eps=cfg.norm_eps))
        self._add_child("attention", cfg.attention.clone(query_dim=d, key_dim=d, value_dim=d, output_dim=d,
                                                         num_heads=cfg.num_heads))
        hidden = int(d * cfg.hidden_dim_scale)
        self._add_child("linear1", Linear.default_config().set(input_dim=d, output_dim=hidden))
        self._add_child("linear2", Linear.default_config().set(input_dim=hidden, output_dim=d))

    def forward(self, inputs: Tensor, *, condition: Tensor) -> Tensor:
        shift_a, scale_a, gate_a, shift_f, scale_f, gate_f = self.adaln(condition)
        h = modulate(self.norm1(inputs), shift=shift_a, scale=scale_a)
        x = inputs + gate_a[:, None] * self.attention(query=h).data
        h = modulate(self.norm2(x), shift=shift_f, scale=scale_f)
        h = self.linear2(get_activation_fn(self._config.activation)(self.linear1(h)))
        return x + gate_f[:, None] * h


class DiTFinalLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        norm_eps: float = 1e-6

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("adaln", AdaptiveLayerNormModulation.default_config().set(dim=cfg.input_dim, num_outputs=2))
        self._add_child("norm", LayerNormStateless.default_config().set(input_dim=cfg.input_dim, eps=cfg.norm_eps))
        self._add_child("linear", Linear.default_config().set(input_dim=cfg.input_dim, output_dim=cfg.output_dim,
                                                              param_init=_zero_init()))

    def forward(self, inputs: Tensor, *, condition: Tensor) -> Tensor:
        shift, scale = self.adaln(condition)
        return self.linear(modulate(self.norm(inputs), shift=shift, scale=scale))


class DiT(BaseLayer):
    """Latent images ``[B, H, W, C]`` + time steps (+ class labels) -> predicted noise (and
    optionally its variance: ``output_channels = 2 * C``) of the same spatial size."""

    @config_class
    class Config(BaseLayer.Config):
        image_size: tuple = (32, 32)
        patch_size: int = 2
        input_channels: int = 4
        output_channels: Optional[int] = None
        dim: Required[int] = REQUIRED
        num_layers: Required[int] = REQUIRED
        num_heads: Required[int] = REQUIRED
        num_classes: Optional[int] = None
        block: InstantiableConfig = DiTBlock.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        p = cfg.patch_size
        self._grid = (cfg.image_size[0] // p, cfg.image_size[1] // p)
        self._out_channels = cfg.output_channels or cfg.input_channels
        self._add_child("patch_emb", Linear.default_config().set(input_dim=p * p * cfg.input_channels, output_dim=cfg.dim))
        self._add_child("time_emb", TimeStepEmbedding.default_config().set(output_dim=cfg.dim))
        if cfg.num_classes is not None:
            self._add_child("label_emb", LabelEmbedding.default_config().set(num_classes=cfg.num_classes, output_dim=cfg.dim))
        self._blocks = [self._add_child(f"block{i}", cfg.block.clone(input_dim=cfg.dim, num_heads=cfg.num_heads))
                        for i in range(cfg.num_layers)]
        self._add_child("final", DiTFinalLayer.default_config().set(input_dim=cfg.dim, output_dim=p * p * self._out_channels))

    def _positions(self, device) -> Tensor:
        """Fixed 2-D sin-cos position embeddings ``[grid_h * grid_w, dim]``."""
        d = self._config.dim // 2

        def one(n):
            pos = torch.arange(n, device=device).float()
            omega = 1.0 / 10000 ** (torch.arange(d // 2, device=device).float() / (d // 2))
            out = pos[:, None] * omega[None]
            return torch.cat([torch.sin(out), torch.cos(out)], dim=-1)

        eh, ew = one(self._grid[0]), one(self._grid[1])
        grid = torch.cat([eh[:, None].expand(-1, self._grid[1], -1), ew[None].expand(self._grid[0], -1, -1)], dim=-1)
        return grid.reshape(-1, grid.shape[-1])

    def forward(self, image: Tensor, *, timesteps: Tensor, labels: Optional[Tensor] = None) -> Tensor:
        cfg = self._config
        b, h, w, c = image.shape
        p, (gh, gw) = cfg.patch_size, self._grid
        patches = image.reshape(b, gh, p, gw, p, c).permute(0, 1, 3, 2, 4, 5).reshape(b, gh * gw, p * p * c)
        x = self.patch_emb(patches)
        pos = self._positions(image.device)
        x = x + torch.nn.functional.pad(pos, (0, cfg.dim - pos.shape[-1])).to(x.dtype)[None]
        cond = self.time_emb(timesteps)
        if labels is not None and "label_emb" in self._children:
            cond = cond + self.label_emb(labels)
        for block in self._blocks:
            x = block(x, condition=cond)
        y = self.final(x, condition=cond)
        oc = self._out_channels
        return y.reshape(b, gh, gw, p, p, oc).permute(0, 1, 3, 2, 4, 5).reshape(b, h, w, oc)
