"""Convolutional subsampling of filterbank features.

Parity target in the reference: axlearn/audio/subsamplers.py (``ConvSubSampler`` :20: two
``Conv2DWith1DPadding`` layers, window 3, stride 2, each followed by an optional norm and an
activation; 4x reduction in time and frequency).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2DWith1DPadding
from axlearn_b200.common.layers import get_activation_fn
from axlearn_b200.common.module import nowrap

Tensor = torch.Tensor


class ConvSubSampler(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: int = 1
        output_dim: Required[int] = REQUIRED
        hidden_dim: Optional[int] = None
        conv: InstantiableConfig = Conv2DWith1DPadding.default_config().set(
            window=(3, 3), strides=(2, 2), padding=((1, 1), (1, 1)))
        norm: Optional[InstantiableConfig] = None
        activation: Optional[str] = "nn.relu"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        hidden = cfg.hidden_dim or cfg.output_dim
        self._add_child("conv1", cfg.conv.clone(input_dim=cfg.input_dim, output_dim=hidden))
        self._add_child("conv2", cfg.conv.clone(input_dim=hidden, output_dim=cfg.output_dim))
        if cfg.norm is not None:
            self._add_child("norm1", cfg.norm.clone(input_dim=hidden))
            self._add_child("norm2", cfg.norm.clone(input_dim=cfg.output_dim))

    @nowrap
    def output_shape(self, *, input_shape: Sequence[Optional[int]]):
        shape = self.conv1.output_shape(input_shape=input_shape)
        return self.conv2.output_shape(input_shape=shape)

    def forward(self, inputs: Tensor, *, paddings: Tensor):
        act = get_activation_fn(self._config.activation) if self._config.activation else (lambda v: v)
        x, p = self.conv1(inputs, paddings=paddings)
        if "norm1" in self._children:
            x = self.norm1(x)
        x = act(x) * (1 - p)[:, :, None, None].to(x.dtype)
        x, p = self.conv2(x, paddings=p)
        if "norm2" in self._children:
            x = self.norm2(x)
        x = act(x) * (1 - p)[:, :, None, None].to(x.dtype)
        return {"outputs": x, "paddings": p}
