"""SpecAugment: random frequency and time masks on filterbank features.

Parity target in the reference: axlearn/audio/spectrum_augmenter.py (``MaskSampler`` :22 -- up
to ``max_num_masks`` masks (or ``max_num_masks_ratio * length``), each of random width up to
``max_mask_length`` (or ratio) -- and ``SpectrumAugmenter`` :132, active only in training).
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import InstantiableConfig, config_class

Tensor = torch.Tensor


class MaskSampler(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        max_num_masks: Optional[int] = None
        max_num_masks_ratio: Optional[float] = None
        max_mask_length: Optional[int] = None
        max_mask_length_ratio: Optional[float] = None

    def forward(self, *, input_lengths: Tensor, max_length: int) -> Tensor:
        """``[B, max_length]`` with 1 where masked.  ``input_lengths [B]`` bounds the positions and,
        with the ratio options, the number and width of the masks."""
        cfg = self._config
        if (cfg.max_num_masks is None) == (cfg.max_num_masks_ratio is None):
            raise ValueError("set exactly one of max_num_masks and max_num_masks_ratio")
        if (cfg.max_mask_length is None) == (cfg.max_mask_length_ratio is None):
            raise ValueError("set exactly one of max_mask_length and max_mask_length_ratio")
        b = input_lengths.shape[0]
        dev = input_lengths.device
        lengths = input_lengths.float()
        if cfg.max_num_masks is not None:
            cap = cfg.max_num_masks
            num_masks = torch.full((b,), cap, device=dev)
        else:
            cap = max(1, int(cfg.max_num_masks_ratio * max_length))
            num_masks = torch.clamp((lengths * cfg.max_num_masks_ratio).long(), max=cap)
        max_len = (torch.full((b,), float(cfg.max_mask_length), device=dev) if cfg.max_mask_length is not None
                   else lengths * cfg.max_mask_length_ratio)
        k1, k2 = prng.split(self.prng_key, 2)
        widths = (prng.uniform(k1, (b, cap), device=dev) * (max_len[:, None] + 1)).floor()
        widths = torch.minimum(widths, lengths[:, None])
        starts = (prng.uniform(k2, (b, cap), device=dev) * (lengths[:, None] - widths + 1)).floor()
        pos = torch.arange(max_length, device=dev)[None, None, :]
        live = torch.arange(cap, device=dev)[None, :] < num_masks[:, None]
        inside = (pos >= starts[..., None]) & (pos < (starts + widths)[..., None]) & live[..., None]
        return inside.any(dim=1).float()


class SpectrumAugmenter(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        freq_mask_sampler: InstantiableConfig = MaskSampler.default_config()
        time_mask_sampler: InstantiableConfig = MaskSampler.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("freq_mask_sampler", cfg.freq_mask_sampler)
        self._add_child("time_mask_sampler", cfg.time_mask_sampler)

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> Tensor:
        """``inputs [B, T, F, C]``; masked cells become 0.  Identity outside training."""
        if not self.is_training:
            return inputs
        b, t, f = inputs.shape[:3]
        lengths = (1 - paddings).sum(dim=1)
        time_mask = self.time_mask_sampler(input_lengths=lengths, max_length=t)
        freq_mask = self.freq_mask_sampler(input_lengths=torch.full((b,), f, device=inputs.device), max_length=f)
        keep = (1 - time_mask)[:, :, None, None] * (1 - freq_mask)[:, None, :, None]
        return inputs * keep.to(inputs.dtype)
