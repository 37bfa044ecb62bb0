"""ResNet backbones (channels-last images ``[B, H, W, C]``).

Parity target in the reference: axlearn/vision/resnet.py (``ConvBatchNormLayer`` :30, ``StemV0``
/ ``StemV1`` :70-140, ``ResidualBlock`` :143, ``BottleneckBlock`` :226, ``ResNetStage`` :320,
``ResNet`` :390 with ``resnet{18,34,50,101,152}`` configs; endpoints named by log2 of the stride:
``"2"`` ... ``"5"``, plus ``"embedding"`` = global average of the last).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.layers import BatchNorm, SqueezeExcitation, StochasticDepth, get_activation_fn

Tensor = torch.Tensor


class ConvBatchNormLayer(BaseLayer):
    """``norm(conv(x))`` with children ``conv`` and ``norm`` (used for the shortcut projection)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        conv: InstantiableConfig = Conv2D.default_config().set(window=(3, 3), padding="SAME", bias=False)
        norm: InstantiableConfig = BatchNorm.default_config().set(decay=0.9, eps=1e-5)
        activation: Optional[str] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("conv", cfg.conv.clone(input_dim=cfg.input_dim, output_dim=cfg.output_dim))
        self._add_child("norm", cfg.norm.clone(input_dim=cfg.output_dim))

    def forward(self, x: Tensor) -> Tensor:
        x = self.norm(self.conv(x))
        return get_activation_fn(self._config.activation)(x) if self._config.activation else x


def _conv_cfg(window: int, strides: int) -> Conv2D.Config:
    return Conv2D.default_config().set(window=(window, window), strides=(strides, strides), padding="SAME", bias=False)


def _norm_cfg() -> BatchNorm.Config:
    return BatchNorm.default_config().set(decay=0.9, eps=1e-5)


def _conv_bn(window, strides, activation=None) -> ConvBatchNormLayer.Config:
    cfg = ConvBatchNormLayer.default_config().set(activation=activation)
    cfg.conv.set(window=(window, window), strides=(strides, strides))
    return cfg


def _max_pool_3x3_s2(x: Tensor) -> Tensor:
    return F.max_pool2d(x.movedim(-1, 1), kernel_size=3, stride=2, padding=1).movedim(1, -1)


class StemV0(BaseLayer):
    """7x7 stride-2 convolution (``conv1``) + batch norm (``norm1``) + ReLU + 3x3 stride-2 max pool."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: int = 3
        hidden_dim: Required[int] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("conv1", _conv_cfg(7, 2).set(input_dim=cfg.input_dim, output_dim=cfg.hidden_dim))
        self._add_child("norm1", _norm_cfg().set(input_dim=cfg.hidden_dim))

    def forward(self, x: Tensor) -> Tensor:
        return _max_pool_3x3_s2(F.relu(self.norm1(self.conv1(x))))


class ResidualBlock(BaseLayer):
    """Two 3x3 convolutions (ResNet-18 / 34): children ``conv1, norm1, conv2, norm2`` and, where the
    shape changes, ``downsample`` (1x1 convolution + norm on the shortcut)."""

    EXPANSION = 1

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        stride: int = 1
        squeeze_excitation: Optional[InstantiableConfig] = None
        stochastic_depth: InstantiableConfig = StochasticDepth.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._num_convs = 0
        self._build_branch()
        if cfg.stride != 1 or cfg.input_dim != cfg.output_dim:
            self._add_child("downsample", _conv_bn(1, cfg.stride).set(input_dim=cfg.input_dim, output_dim=cfg.output_dim))
        if cfg.squeeze_excitation is not None:
            self._add_child("squeeze_excitation", cfg.squeeze_excitation.clone(input_dim=cfg.output_dim))
        self._add_child("stochastic_depth", cfg.stochastic_depth)

    def _add_conv(self, window: int, stride: int, input_dim: int, output_dim: int) -> None:
        self._num_convs += 1
        i = self._num_convs
        self._add_child(f"conv{i}", _conv_cfg(window, stride).set(input_dim=input_dim, output_dim=output_dim))
        self._add_child(f"norm{i}", _norm_cfg().set(input_dim=output_dim))

    def _build_branch(self):
        cfg = self._config
        self._add_conv(3, cfg.stride, cfg.input_dim, cfg.output_dim)
        self._add_conv(3, 1, cfg.output_dim, cfg.output_dim)

    def forward(self, x: Tensor) -> Tensor:
        y = x
        for i in range(1, self._num_convs + 1):
            y = getattr(self, f"norm{i}")(getattr(self, f"conv{i}")(y))
            if i < self._num_convs:
                y = F.relu(y)
        if "squeeze_excitation" in self._children:
            y = self.squeeze_excitation(y)
        skip = self.downsample(x) if "downsample" in self._children else x
        return F.relu(skip + self.stochastic_depth(y))


class BottleneckBlock(ResidualBlock):
    """1x1 reduce, 3x3 (carrying the stride), 1x1 expand by 4 (ResNet-50 and deeper)."""

    EXPANSION = 4

    def _build_branch(self):
        cfg = self._config
        mid = cfg.output_dim // self.EXPANSION
        self._add_conv(1, 1, cfg.input_dim, mid)
        self._add_conv(3, cfg.stride, mid, mid)
        self._add_conv(1, 1, mid, cfg.output_dim)


class ResNetStage(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        num_blocks: Required[int] = REQUIRED
        stride: int = 1
        block: InstantiableConfig = BottleneckBlock.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._blocks = []
        for i in range(cfg.num_blocks):
            self._blocks.append(self._add_child(f"block{i}", cfg.block.clone(
                input_dim=cfg.input_dim if i == 0 else cfg.output_dim, output_dim=cfg.output_dim,
                stride=cfg.stride if i == 0 else 1)))

    def forward(self, x: Tensor) -> Tensor:
        for b in self._blocks:
            x = b(x)
        return x


class ResNet(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        stem: InstantiableConfig = StemV0.default_config()
        stage: InstantiableConfig = ResNetStage.default_config()
        hidden_dim: int = 64
        num_blocks_per_stage: Sequence[int] = (3, 4, 6, 3)
        # Peak stochastic-depth rate, growing linearly over the blocks (None = off).
        peak_stochastic_depth_rate: Optional[float] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("stem", cfg.stem.clone(hidden_dim=cfg.hidden_dim))
        expansion = cfg.stage.block.klass.EXPANSION
        dim_in = cfg.hidden_dim
        self._stages = []
        self._endpoint_dims = {}
        for i, n in enumerate(cfg.num_blocks_per_stage):
            dim_out = cfg.hidden_dim * (2 ** i) * expansion
            stage = cfg.stage.clone(input_dim=dim_in, output_dim=dim_out, num_blocks=n, stride=1 if i == 0 else 2)
            if cfg.peak_stochastic_depth_rate:
                stage.block.stochastic_depth.rate = cfg.peak_stochastic_depth_rate * (i + 1) / len(cfg.num_blocks_per_stage)
            self._stages.append(self._add_child(f"stage{i}", stage))
            self._endpoint_dims[str(i + 2)] = dim_out
            dim_in = dim_out
        self._endpoint_dims["embedding"] = dim_in

    @property
    def endpoints_dims(self) -> dict:
        return dict(self._endpoint_dims)

    def forward(self, image: Tensor) -> dict:
        x = self.stem(image)
        endpoints = {}
        for i, stage in enumerate(self._stages):
            x = stage(x)
            endpoints[str(i + 2)] = x
        endpoints["embedding"] = x.mean(dim=(1, 2))
        return endpoints


def named_resnet_config(name: str) -> ResNet.Config:
    table = {"resnet18": (ResidualBlock, (2, 2, 2, 2)), "resnet34": (ResidualBlock, (3, 4, 6, 3)),
             "resnet50": (BottleneckBlock, (3, 4, 6, 3)), "resnet101": (BottleneckBlock, (3, 4, 23, 3)),
             "resnet152": (BottleneckBlock, (3, 8, 36, 3))}
    block, blocks = table[name]
    cfg = ResNet.default_config().set(num_blocks_per_stage=blocks)
    cfg.stage.block = block.default_config()
    return cfg
