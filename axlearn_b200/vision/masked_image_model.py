"""Masked image modelling (BEiT / MAE style): block-wise mask generator, target tokenizers, a ViT
encoder with a mask token, and the model that predicts the targets of the masked patches.

Reference: axlearn/vision/mask_generator.py (``MaskingGenerator``), beit_image_tokenizer.py (a
frozen discrete tokenizer), feature_tokenizer.py, masked_image_model.py (``MaskedImageModel``
:27-151).  Targets are either vocabulary ids (cross-entropy) or per-patch features (regression);
only masked positions count.
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from axlearn_b200.common import prng
from axlearn_b200.common.attention import StackedTransformerLayer
from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.embedding import LearnedPositionalEmbedding
from axlearn_b200.common.layers import LayerNorm, Linear
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.param_init import gaussian_initializer

Tensor = torch.Tensor


class MaskingGenerator:
    """Block-wise masking: rectangles of random area and aspect ratio are added until
    ``num_masking_patches`` cells of the ``[height, width]`` patch grid are masked."""

    def __init__(self, *, input_size: tuple, num_masking_patches: int, min_mask_patches: int = 4,
                 max_mask_patches: Optional[int] = None, min_aspect: float = 0.3, max_aspect: Optional[float] = None,
                 max_attempts: int = 10):
        self.height, self.width = input_size
        self.num_masking_patches = num_masking_patches
        self.min_mask_patches = min_mask_patches
        self.max_mask_patches = num_masking_patches if max_mask_patches is None else max_mask_patches
        max_aspect = max_aspect or 1 / min_aspect
        self.log_aspect = (math.log(min_aspect), math.log(max_aspect))
        self.max_attempts = max_attempts

    def _add_block(self, mask: np.ndarray, budget: int, rng: np.random.Generator) -> int:
        for _ in range(self.max_attempts):
            area = rng.uniform(self.min_mask_patches, max(self.min_mask_patches, budget))
            aspect = math.exp(rng.uniform(*self.log_aspect))
            h, w = int(round(math.sqrt(area * aspect))), int(round(math.sqrt(area / aspect)))
            if not (0 < h <= self.height and 0 < w <= self.width):
                continue
            top, left = rng.integers(0, self.height - h + 1), rng.integers(0, self.width - w + 1)
            new = h * w - int(mask[top:top + h, left:left + w].sum())
            if 0 < new <= budget:
                mask[top:top + h, left:left + w] = True
                return new
        return 0

    def __call__(self, seed: int = 0) -> np.ndarray:
        rng = np.random.default_rng(seed)
        mask = np.zeros((self.height, self.width), dtype=bool)
        count = 0
        while count < self.num_masking_patches:
            added = self._add_block(mask, min(self.num_masking_patches - count, self.max_mask_patches), rng)
            if added == 0:
                break
            count += added
        # Top up with single cells so that every example masks exactly the same number of patches.
        if count < self.num_masking_patches:
            free = np.flatnonzero(~mask.reshape(-1))
            mask.reshape(-1)[rng.choice(free, self.num_masking_patches - count, replace=False)] = True
        return mask


def patchify(image: Tensor, patch_size: tuple) -> Tensor:
    """``[B, H, W, C] -> [B, (H/p)(W/q), p*q*C]``."""
    b, h, w, c = image.shape
    p, q = patch_size
    x = image.reshape(b, h // p, p, w // q, q, c).permute(0, 1, 3, 2, 4, 5)
    return x.reshape(b, (h // p) * (w // q), p * q * c)


class PatchFeatureTokenizer(BaseLayer):
    """Regression targets: the pixels of every patch, optionally normalised per patch (MAE)."""

    @config_class
    class Config(BaseLayer.Config):
        patch_size: tuple = (16, 16)
        normalize: bool = True

    def forward(self, image: Tensor) -> Tensor:
        x = patchify(image.float(), self._config.patch_size)
        if self._config.normalize:
            x = (x - x.mean(-1, keepdim=True)) / (x.var(-1, keepdim=True) + 1e-6).sqrt()
        return x


class DiscreteImageTokenizer(BaseLayer):
    """Classification targets: a strided convolutional encoder whose outputs are matched to the
    nearest of ``vocab_size`` codebook vectors (the role of BEiT's frozen dVAE tokenizer).  It is
    evaluated without gradients; its weights come from a checkpoint or stay at their random
    initialisation (a fixed random tokenizer is already a usable pretext task)."""

    @config_class
    class Config(BaseLayer.Config):
        patch_size: tuple = (16, 16)
        num_channels: int = 3
        hidden_dim: int = 64
        vocab_size: int = 8192

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", Conv2D.default_config().set(
            window=cfg.patch_size, strides=cfg.patch_size, input_dim=cfg.num_channels, output_dim=cfg.hidden_dim))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"codebook": ParameterSpec(shape=(cfg.vocab_size, cfg.hidden_dim), mesh_axes=(None, None),
                                          initializer=gaussian_initializer(1.0))}

    @torch.no_grad()
    def forward(self, image: Tensor) -> Tensor:
        z = self.encoder(image.float())
        z = z.reshape(z.shape[0], -1, z.shape[-1])
        code = self.parameters["codebook"].float()
        d = (z ** 2).sum(-1, keepdim=True) - 2 * z @ code.t() + (code ** 2).sum(-1)[None, None]
        return d.argmin(dim=-1)


class MaskedImageEncoder(BaseLayer):
    """ViT over patches where masked patches are replaced by a learned mask token."""

    @config_class
    class Config(BaseLayer.Config):
        image_size: tuple = (224, 224)
        patch_size: tuple = (16, 16)
        num_channels: int = 3
        dim: Required[int] = REQUIRED
        transformer: InstantiableConfig = StackedTransformerLayer.default_config()
        output_norm: InstantiableConfig = LayerNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("patch_emb", Conv2D.default_config().set(
            window=cfg.patch_size, strides=cfg.patch_size, input_dim=cfg.num_channels, output_dim=cfg.dim))
        self.grid = (cfg.image_size[0] // cfg.patch_size[0], cfg.image_size[1] // cfg.patch_size[1])
        self._add_child("pos_emb", LearnedPositionalEmbedding.default_config().set(dim=cfg.dim, shape=(self.grid[0] * self.grid[1],)))
        self._add_child("transformer", cfg.transformer.clone(input_dim=cfg.dim))
        self._add_child("output_norm", cfg.output_norm.clone(input_dim=cfg.dim))

    def _create_layer_parameter_specs(self):
        return {"mask_token": ParameterSpec(shape=(1, 1, self._config.dim), mesh_axes=(None, None, None),
                                            initializer=gaussian_initializer(0.02))}

    @property
    def endpoints_dims(self) -> dict:
        return {"embedding": self._config.dim}

    def forward(self, image: Tensor, *, is_masked: Optional[Tensor] = None) -> dict:
        x = self.patch_emb(image)
        x = x.reshape(x.shape[0], -1, x.shape[-1])
        if is_masked is not None:
            x = torch.where(is_masked[..., None], self.parameters["mask_token"].to(x.dtype), x)
        x = x + self.pos_emb(torch.arange(x.shape[1], device=x.device)[None])
        x = self.output_norm(self.transformer(x).data)
        return {"encoded_features": x, "embedding": x.mean(dim=1)}


class MaskedImageModel(BaseModel):
    """``input_batch = {"image": [B, H, W, C], "is_masked": [B, patches] bool}``; without
    ``is_masked`` a block-wise mask is drawn per example."""

    @config_class
    class Config(BaseModel.Config):
        tokenizer: Required[InstantiableConfig] = REQUIRED
        encoder: Required[InstantiableConfig] = REQUIRED
        head: InstantiableConfig = Linear.default_config().set(bias=True)
        mask_ratio: float = 0.4

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("tokenizer", cfg.tokenizer)
        self._add_child("encoder", cfg.encoder)
        tok = cfg.tokenizer
        if "vocab_size" in tok.keys():
            out_dim = tok.vocab_size
        else:
            out_dim = tok.patch_size[0] * tok.patch_size[1] * cfg.encoder.num_channels
        self._add_child("head", cfg.head.clone(input_dim=self.encoder.endpoints_dims["embedding"], output_dim=out_dim))

    def generate_labels(self, image: Tensor) -> Tensor:
        return self.tokenizer(image).detach()

    def _draw_masks(self, batch: int, device) -> Tensor:
        grid = self.encoder.grid
        gen = MaskingGenerator(input_size=grid, num_masking_patches=max(1, int(self._config.mask_ratio * grid[0] * grid[1])),
                               min_mask_patches=min(4, max(1, grid[0] * grid[1] // 8)))
        base = int(prng.randint(self.prng_key, (), 0, 2 ** 31 - 1)) if self.prng_key is not None else 0
        masks = np.stack([gen(base + i).reshape(-1) for i in range(batch)])
        return torch.from_numpy(masks).to(device)

    def predict(self, input_batch: dict) -> dict:
        image = input_batch["image"]
        is_masked = input_batch.get("is_masked")
        if is_masked is None:
            is_masked = self._draw_masks(image.shape[0], image.device)
        enc = self.encoder(image, is_masked=is_masked.bool())
        return {"logits": self.head(enc["encoded_features"]), "is_masked": is_masked.bool(), **enc}

    def forward(self, input_batch: dict):
        out = self.predict(input_batch)
        labels = self.generate_labels(input_batch["image"])
        live = out["is_masked"]
        n = live.sum().clamp_min(1)
        pred = out["logits"].float()
        if labels.dtype in (torch.int64, torch.int32):
            per = F.cross_entropy(pred.reshape(-1, pred.shape[-1]), labels.reshape(-1), reduction="none").reshape(labels.shape)
            acc = ((pred.argmax(-1) == labels) & live).sum() / n
            self.add_summary("accuracy", WeightedSummary(acc, n))
        else:
            per = ((pred - labels) ** 2).mean(-1)
        loss = (per * live).sum() / n
        self.add_summary("loss", WeightedSummary(loss.detach(), n))
        return loss, {"labels": labels, **out}
