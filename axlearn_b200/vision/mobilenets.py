"""MobileNetV3 and EfficientNet (V1 / lite / V2) backbones from one block vocabulary.

Reference: axlearn/vision/mobilenets_blocks.py (``ConvBnAct`` :141, ``MobileBlock`` :204-405) and
axlearn/vision/mobilenets.py (``MobileNets`` :235, block-string decoding :523, architecture tables
:654 and :810, ``named_model_configs`` :951).

A network is a stem convolution, stages of blocks and an embedding head.  Blocks: ``conv`` (conv +
norm + activation), ``ds`` (depthwise-separable), ``ir`` (inverted residual: expand 1x1, depthwise,
squeeze-excite, project 1x1) and ``fir`` (fused inverted residual: the expansion and the depthwise
convolution are one dense convolution).  Stages are written as rows of
``(block, repeats, kernel, stride, expansion, channels, se_ratio, activation)``; width and depth
multipliers scale channels (rounded to multiples of 8) and repeats (rounded up).  The forward pass
returns endpoints keyed by stride level (``"1"`` ... ``"5"``) plus ``"embedding"``.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.layers import (
    BatchNorm,
    Linear,
    SqueezeExcitation,
    StochasticDepth,
    get_activation_fn,
)

Tensor = torch.Tensor


def make_divisible(value: float, divisor: int = 8, min_value: Optional[int] = None, round_limit: float = 0.9) -> int:
    """Rounds to a multiple of ``divisor`` without dropping below ``round_limit * value``."""
    min_value = min_value or divisor
    new = max(min_value, int(value + divisor / 2) // divisor * divisor)
    return new + divisor if new < round_limit * value else new


def round_features(features: int, multiplier: float = 1.0, divisor: int = 8) -> int:
    return features if not multiplier else make_divisible(features * multiplier, divisor)


def _same_conv(window: int, stride: int, groups: int = 1) -> InstantiableConfig:
    pad = (window - 1) // 2
    return Conv2D.default_config().set(window=(window, window), strides=(stride, stride),
                                       padding=((pad, window - 1 - pad),) * 2, bias=False,
                                       num_input_dim_groups=groups)


class ConvBnAct(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        window: int = 1
        stride: int = 1
        depthwise: bool = False
        norm: Optional[InstantiableConfig] = BatchNorm.default_config()
        activation: Optional[str] = "nn.relu"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        groups = cfg.input_dim if cfg.depthwise else 1
        self._add_child("conv", _same_conv(cfg.window, cfg.stride, groups).set(
            input_dim=cfg.input_dim, output_dim=cfg.output_dim))
        if cfg.norm is not None:
            self._add_child("bn", cfg.norm.clone(input_dim=cfg.output_dim))

    def forward(self, x: Tensor) -> Tensor:
        x = self.conv(x)
        if "bn" in self._children:
            x = self.bn(x)
        act = self._config.activation
        return get_activation_fn(act)(x) if act else x


class MobileBlock(BaseLayer):
    """One ``conv`` / ``ds`` / ``ir`` / ``fir`` block with an identity shortcut when shapes allow."""

    @config_class
    class Config(BaseLayer.Config):
        block_type: str = "ir"
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        window: int = 3
        stride: int = 1
        exp_ratio: float = 1.0
        se_ratio: float = 0.0
        # Squeeze width relative to the block input (EfficientNet) or to the expanded width
        # (MobileNetV3).
        se_reduce_from_input: bool = True
        se_gating: str = "nn.sigmoid"
        activation: str = "nn.relu"
        drop_path_rate: Optional[float] = None
        norm: InstantiableConfig = BatchNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        kind = cfg.block_type
        if kind not in ("conv", "ds", "ir", "fir"):
            raise ValueError(f"unknown block type {kind}")
        mid = make_divisible(cfg.input_dim * cfg.exp_ratio) if kind in ("ir", "fir") else cfg.input_dim
        self._mid = mid

        def cba(name, **kw):
            self._add_child(name, ConvBnAct.default_config().set(norm=cfg.norm.clone(), **kw))

        if kind == "conv":
            cba("conv", input_dim=cfg.input_dim, output_dim=cfg.output_dim, window=cfg.window, stride=cfg.stride,
                activation=cfg.activation)
        elif kind == "ds":
            cba("dw", input_dim=cfg.input_dim, output_dim=cfg.input_dim, window=cfg.window, stride=cfg.stride,
                depthwise=True, activation=cfg.activation)
        elif kind == "ir":
            if mid != cfg.input_dim or cfg.exp_ratio != 1.0:
                cba("expand", input_dim=cfg.input_dim, output_dim=mid, activation=cfg.activation)
            cba("dw", input_dim=mid, output_dim=mid, window=cfg.window, stride=cfg.stride, depthwise=True,
                activation=cfg.activation)
        else:
            cba("expand", input_dim=cfg.input_dim, output_dim=mid, window=cfg.window, stride=cfg.stride,
                activation=cfg.activation)
        if kind != "conv":
            if cfg.se_ratio > 0:
                base = cfg.input_dim if cfg.se_reduce_from_input else mid
                self._add_child("se", SqueezeExcitation.default_config().set(
                    input_dim=mid, se_ratio=cfg.se_ratio, gating=cfg.se_gating,
                    activation="nn.relu" if not cfg.se_reduce_from_input else cfg.activation,
                    num_reduced_filters=make_divisible(base * cfg.se_ratio) if not cfg.se_reduce_from_input
                    else max(1, int(base * cfg.se_ratio))))
            cba("project", input_dim=mid, output_dim=cfg.output_dim, activation=None)
        self._residual = cfg.stride == 1 and cfg.input_dim == cfg.output_dim and kind != "conv"
        if self._residual:
            self._add_child("drop_path", StochasticDepth.default_config().set(rate=cfg.drop_path_rate))

    def forward(self, x: Tensor) -> Tensor:
        y = x
        for name in ("conv", "expand", "dw", "se", "project"):
            if name in self._children:
                y = getattr(self, name)(y)
        return x + self.drop_path(y) if self._residual else y


# (block, repeats, kernel, stride, expansion, channels, se_ratio, activation)
_V3_LARGE = [
    [("ds", 1, 3, 1, 1, 16, 0, "nn.relu")],
    [("ir", 1, 3, 2, 4, 24, 0, "nn.relu"), ("ir", 1, 3, 1, 3, 24, 0, "nn.relu")],
    [("ir", 3, 5, 2, 3, 40, 0.25, "nn.relu")],
    [("ir", 1, 3, 2, 6, 80, 0, "nn.hard_swish"), ("ir", 1, 3, 1, 2.5, 80, 0, "nn.hard_swish"),
     ("ir", 2, 3, 1, 2.3, 80, 0, "nn.hard_swish")],
    [("ir", 2, 3, 1, 6, 112, 0.25, "nn.hard_swish")],
    [("ir", 3, 5, 2, 6, 160, 0.25, "nn.hard_swish")],
    [("conv", 1, 1, 1, 1, 960, 0, "nn.hard_swish")],
]
_V3_SMALL = [
    [("ds", 1, 3, 2, 1, 16, 0.25, "nn.relu")],
    [("ir", 1, 3, 2, 4.5, 24, 0, "nn.relu"), ("ir", 1, 3, 1, 3.67, 24, 0, "nn.relu")],
    [("ir", 1, 5, 2, 4, 40, 0.25, "nn.hard_swish"), ("ir", 2, 5, 1, 6, 40, 0.25, "nn.hard_swish")],
    [("ir", 2, 5, 1, 3, 48, 0.25, "nn.hard_swish")],
    [("ir", 3, 5, 2, 6, 96, 0.25, "nn.hard_swish")],
    [("conv", 1, 1, 1, 1, 576, 0, "nn.hard_swish")],
]
_EFFICIENTNET_B0 = [
    [("ds", 1, 3, 1, 1, 16, 0.25, "nn.swish")],
    [("ir", 2, 3, 2, 6, 24, 0.25, "nn.swish")],
    [("ir", 2, 5, 2, 6, 40, 0.25, "nn.swish")],
    [("ir", 3, 3, 2, 6, 80, 0.25, "nn.swish")],
    [("ir", 3, 5, 1, 6, 112, 0.25, "nn.swish")],
    [("ir", 4, 5, 2, 6, 192, 0.25, "nn.swish")],
    [("ir", 1, 3, 1, 6, 320, 0.25, "nn.swish")],
]
_EFFICIENTNET_V2_S = [
    [("conv", 2, 3, 1, 1, 24, 0, "nn.swish")],
    [("fir", 4, 3, 2, 4, 48, 0, "nn.swish")],
    [("fir", 4, 3, 2, 4, 64, 0, "nn.swish")],
    [("ir", 6, 3, 2, 4, 128, 0.25, "nn.swish")],
    [("ir", 9, 3, 1, 6, 160, 0.25, "nn.swish")],
    [("ir", 15, 3, 2, 6, 256, 0.25, "nn.swish")],
]
# (width multiplier, depth multiplier, input resolution) of EfficientNet B0 ... B7.
_EFFICIENTNET_SCALES = {
    "B0": (1.0, 1.0, 224), "B1": (1.0, 1.1, 240), "B2": (1.1, 1.2, 260), "B3": (1.2, 1.4, 300),
    "B4": (1.4, 1.8, 380), "B5": (1.6, 2.2, 456), "B6": (1.8, 2.6, 528), "B7": (2.0, 3.1, 600),
}


class MobileNets(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        stages: Required[Sequence] = REQUIRED          # rows as in the tables above
        stem_dim: int = 16
        stem_activation: str = "nn.hard_swish"
        width_multiplier: float = 1.0
        depth_multiplier: float = 1.0
        fix_first_last: bool = False                    # EfficientNet-lite keeps stem / last stage depth
        se_reduce_from_input: bool = True
        se_gating: str = "nn.sigmoid"
        embedding_dim: Optional[int] = None            # a final 1x1 conv (EfficientNet) or linear (V3)
        embedding_kind: str = "conv"
        embedding_activation: str = "nn.swish"
        peak_stochastic_depth_rate: Optional[float] = None
        norm: InstantiableConfig = BatchNorm.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        stem_dim = round_features(cfg.stem_dim, cfg.width_multiplier)
        self._add_child("stem", ConvBnAct.default_config().set(
            input_dim=3, output_dim=stem_dim, window=3, stride=2, activation=cfg.stem_activation, norm=cfg.norm.clone()))
        total = sum(self._repeats(rep, si, len(cfg.stages)) for si, rows in enumerate(cfg.stages) for (_, rep, *_r) in rows)
        dim, level, index = stem_dim, 1, 0
        self._blocks: list[tuple[str, int]] = []
        self._endpoint_dims = {"1": stem_dim}
        for si, rows in enumerate(cfg.stages):
            for ri, (kind, rep, window, stride, exp, channels, se, act) in enumerate(rows):
                out_dim = round_features(channels, cfg.width_multiplier)
                for r in range(self._repeats(rep, si, len(cfg.stages))):
                    s = stride if r == 0 else 1
                    if s == 2:
                        self._endpoint_dims[str(level)] = dim
                        level += 1
                    name = f"stage{si}_block{ri}_{r}"
                    rate = cfg.peak_stochastic_depth_rate * index / total if cfg.peak_stochastic_depth_rate else None
                    self._add_child(name, MobileBlock.default_config().set(
                        block_type=kind, input_dim=dim, output_dim=out_dim, window=window, stride=s, exp_ratio=exp,
                        se_ratio=se, activation=act, drop_path_rate=rate, norm=cfg.norm.clone(),
                        se_reduce_from_input=cfg.se_reduce_from_input, se_gating=cfg.se_gating))
                    self._blocks.append((name, level))
                    dim = out_dim
                    index += 1
        self._endpoint_dims[str(level)] = dim
        self._last_level = level
        if cfg.embedding_dim:
            emb_dim = cfg.embedding_dim if cfg.embedding_kind == "linear" else round_features(
                cfg.embedding_dim, max(1.0, cfg.width_multiplier))
            if cfg.embedding_kind == "conv":
                self._add_child("embedding_conv", ConvBnAct.default_config().set(
                    input_dim=dim, output_dim=emb_dim, activation=cfg.embedding_activation, norm=cfg.norm.clone()))
            else:
                self._add_child("embedding_linear", Linear.default_config().set(input_dim=dim, output_dim=emb_dim))
            dim = emb_dim
        self._endpoint_dims["embedding"] = dim

    def _repeats(self, rep: int, stage: int, num_stages: int) -> int:
        cfg = self._config
        if cfg.fix_first_last and stage in (0, num_stages - 1):
            return rep
        return int(math.ceil(rep * cfg.depth_multiplier))

    @property
    def endpoints_dims(self) -> dict:
        return dict(self._endpoint_dims)

    def forward(self, image: Tensor) -> dict:
        cfg = self._config
        x = self.stem(image)
        endpoints, level = {}, 1
        for name, block_level in self._blocks:
            if block_level != level:
                endpoints[str(level)] = x
                level = block_level
            x = getattr(self, name)(x)
        endpoints[str(level)] = x
        if "embedding_conv" in self._children:
            x = self.embedding_conv(x).mean(dim=(1, 2))
        else:
            x = x.mean(dim=(1, 2))
            if "embedding_linear" in self._children:
                x = get_activation_fn(cfg.embedding_activation)(self.embedding_linear(x))
        endpoints["embedding"] = x
        return endpoints


def named_model_configs(name: str) -> InstantiableConfig:
    """``mobilenetv3-{small,large}-{minimal-,}{075,100}``, ``efficientnet-b0`` ... ``-b7``,
    ``efficientnet-lite0`` ... ``-lite4``, ``efficientnetv2-s``."""
    key = name.lower()
    cfg = MobileNets.default_config()
    if key.startswith("mobilenetv3"):
        parts = key.split("-")
        table = _V3_LARGE if "large" in parts else _V3_SMALL
        width = {"075": 0.75, "100": 1.0}[parts[-1]]
        if "minimal" in parts:       # no squeeze-excite, no hard-swish, 3x3 kernels only
            table = [[(k, r, 3, s, e, c, 0, "nn.relu") for (k, r, _w, s, e, c, _se, _a) in rows] for rows in table]
        return cfg.set(stages=table, stem_dim=16, stem_activation="nn.relu" if "minimal" in parts else "nn.hard_swish",
                       width_multiplier=width, se_reduce_from_input=False, se_gating="nn.hard_sigmoid",
                       embedding_dim=1280 if "large" in parts else 1024, embedding_kind="linear",
                       embedding_activation="nn.relu" if "minimal" in parts else "nn.hard_swish")
    if key.startswith("efficientnetv2"):
        if key != "efficientnetv2-s":
            raise ValueError(f"unknown model {name}")
        return cfg.set(stages=_EFFICIENTNET_V2_S, stem_dim=24, stem_activation="nn.swish", embedding_dim=1280)
    if key.startswith("efficientnet-lite"):
        w, d, _ = list(_EFFICIENTNET_SCALES.values())[int(key[-1])]
        lite = [[(k, r, win, s, e, c, 0, "nn.relu6") for (k, r, win, s, e, c, _se, _a) in rows] for rows in _EFFICIENTNET_B0]
        return cfg.set(stages=lite, stem_dim=32, stem_activation="nn.relu6", width_multiplier=w, depth_multiplier=d,
                       fix_first_last=True, embedding_dim=1280, embedding_activation="nn.relu6")
    if key.startswith("efficientnet-b"):
        w, d, _ = _EFFICIENTNET_SCALES[key[-2:].upper()]
        return cfg.set(stages=_EFFICIENTNET_B0, stem_dim=32, stem_activation="nn.swish", width_multiplier=w,
                       depth_multiplier=d, embedding_dim=1280)
    raise ValueError(f"unknown model {name}")
