"""EfficientDet: a weighted bidirectional feature pyramid (BiFPN) and separable-convolution heads.

Reference: axlearn/vision/fpn.py (``BiFPN`` and its ``WeightedFeatureFusion`` / depthwise-separable
convolutions) and axlearn/vision/efficientdet.py (compound-scaling table and
``set_efficientdet_config``).  The model itself is ``RetinaNetModel`` (same anchors, focal and Huber
losses) with the pyramid and head swapped.

A BiFPN layer runs a top-down pass (level ``l`` = fuse(input_l, up(td_{l+1}))) and a bottom-up pass
(out_l = fuse(input_l, td_l, down(out_{l-1}))); every fusion is a softmax- or fast-normalised
weighted sum with learned scalar weights, followed by swish, a depthwise-separable convolution and
batch norm.  Levels above the backbone's coarsest are made by 1x1 convolution + stride-2 max pool.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.layers import BatchNorm
from axlearn_b200.common.param_init import ConstantInitializer, DefaultInitializer
from axlearn_b200.vision import mobilenets
from axlearn_b200.vision.retinanet import RetinaNetModel, _upsample_nearest

Tensor = torch.Tensor


class SeparableConv(BaseLayer):
    """3x3 depthwise then 1x1 pointwise convolution, optional batch norm."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        norm: Optional[InstantiableConfig] = BatchNorm.default_config()
        pointwise_param_init: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("depthwise", Conv2D.default_config().set(
            window=(3, 3), padding=((1, 1), (1, 1)), bias=False, input_dim=cfg.input_dim, output_dim=cfg.input_dim,
            num_input_dim_groups=cfg.input_dim))
        pw = Conv2D.default_config().set(window=(1, 1), bias=True, input_dim=cfg.input_dim, output_dim=cfg.output_dim)
        if cfg.pointwise_param_init is not None:
            pw.param_init = cfg.pointwise_param_init
        self._add_child("pointwise", pw)
        if cfg.norm is not None:
            self._add_child("norm", cfg.norm.clone(input_dim=cfg.output_dim))

    def forward(self, x: Tensor) -> Tensor:
        x = self.pointwise(self.depthwise(x))
        return self.norm(x) if "norm" in self._children else x


class WeightedFeatureFusion(BaseLayer):
    """``sum_i w_i x_i`` with ``w = softmax(p)`` or ``relu(p) / (sum relu(p) + eps)``."""

    @config_class
    class Config(BaseLayer.Config):
        num_inputs: Required[int] = REQUIRED
        method: str = "fastattention"           # "attention" (softmax) | "fastattention" | "sum"

    def _create_layer_parameter_specs(self):
        cfg = self._config
        if cfg.method == "sum":
            return {}
        return {"fusion_scale": ParameterSpec(shape=(cfg.num_inputs,), mesh_axes=(None,),
                                        initializer=ConstantInitializer.default_config().set(value=1.0).instantiate())}

    def forward(self, xs: Sequence[Tensor]) -> Tensor:
        cfg = self._config
        if cfg.method == "sum":
            return sum(xs)
        p = self.parameters["fusion_scale"].float()
        w = torch.softmax(p, dim=0) if cfg.method == "attention" else F.relu(p) / (F.relu(p).sum() + 1e-4)
        return sum(x * w[i].to(x.dtype) for i, x in enumerate(xs))


def _resize(x: Tensor, size) -> Tensor:
    """Nearest-neighbour upsampling or max-pool downsampling to ``size`` (H, W)."""
    if x.shape[1] < size[0]:
        return _upsample_nearest(x, size)
    if x.shape[1] == size[0]:
        return x
    y = F.max_pool2d(x.permute(0, 3, 1, 2), kernel_size=3, stride=2, padding=1)
    return y.permute(0, 2, 3, 1)


class BiFPNLayer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        hidden_dim: Required[int] = REQUIRED
        min_level: Required[int] = REQUIRED
        max_level: Required[int] = REQUIRED
        fusion_method: str = "fastattention"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        for level in range(cfg.min_level, cfg.max_level):                   # top-down nodes
            self._add_child(f"td_fuse{level}", WeightedFeatureFusion.default_config().set(num_inputs=2, method=cfg.fusion_method))
            self._add_child(f"td_conv{level}", SeparableConv.default_config().set(input_dim=cfg.hidden_dim, output_dim=cfg.hidden_dim))
        for level in range(cfg.min_level + 1, cfg.max_level + 1):           # bottom-up nodes
            n = 2 if level == cfg.max_level else 3
            self._add_child(f"bu_fuse{level}", WeightedFeatureFusion.default_config().set(num_inputs=n, method=cfg.fusion_method))
            self._add_child(f"bu_conv{level}", SeparableConv.default_config().set(input_dim=cfg.hidden_dim, output_dim=cfg.hidden_dim))

    def forward(self, feats: dict) -> dict:
        cfg = self._config
        td = {cfg.max_level: feats[cfg.max_level]}
        for level in range(cfg.max_level - 1, cfg.min_level - 1, -1):
            up = _resize(td[level + 1], feats[level].shape[1:3])
            fused = getattr(self, f"td_fuse{level}")([feats[level], up])
            td[level] = getattr(self, f"td_conv{level}")(F.silu(fused))
        out = {cfg.min_level: td[cfg.min_level]}
        for level in range(cfg.min_level + 1, cfg.max_level + 1):
            down = _resize(out[level - 1], feats[level].shape[1:3])
            inputs = [feats[level], down] if level == cfg.max_level else [feats[level], td[level], down]
            fused = getattr(self, f"bu_fuse{level}")(inputs)
            out[level] = getattr(self, f"bu_conv{level}")(F.silu(fused))
        return out


class BiFPN(BaseLayer):
    """Drop-in for ``FPN``: ``{level: features}`` of the backbone -> ``{level: [B, H, W, hidden]}``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dims: Required[dict] = REQUIRED
        hidden_dim: int = 64
        min_level: int = 3
        max_level: int = 7
        num_layers: int = 3
        fusion_method: str = "fastattention"

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._backbone_levels = sorted(int(k) for k in cfg.input_dims if cfg.min_level <= int(k) <= cfg.max_level)
        dim = None
        for level in range(cfg.min_level, cfg.max_level + 1):
            dim = cfg.input_dims[str(level)] if level in self._backbone_levels else dim
            if level in self._backbone_levels or level == self._backbone_levels[-1] + 1:
                self._add_child(f"resample{level}", Conv2D.default_config().set(window=(1, 1), bias=True, input_dim=dim, output_dim=cfg.hidden_dim))
                self._add_child(f"resample_norm{level}", BatchNorm.default_config().set(input_dim=cfg.hidden_dim))
            dim = cfg.hidden_dim if level >= self._backbone_levels[-1] + 1 else dim
        for i in range(cfg.num_layers):
            self._add_child(f"layer{i}", BiFPNLayer.default_config().set(
                hidden_dim=cfg.hidden_dim, min_level=cfg.min_level, max_level=cfg.max_level, fusion_method=cfg.fusion_method))

    def forward(self, endpoints: dict) -> dict:
        cfg = self._config
        feats = {}
        top = self._backbone_levels[-1]
        for level in range(cfg.min_level, cfg.max_level + 1):
            if level in self._backbone_levels:
                x = endpoints[str(level)]
                feats[level] = getattr(self, f"resample_norm{level}")(getattr(self, f"resample{level}")(x))
            elif level == top + 1:
                x = getattr(self, f"resample_norm{level}")(getattr(self, f"resample{level}")(endpoints[str(top)]))
                feats[level] = _resize(x, ((x.shape[1] + 1) // 2, (x.shape[2] + 1) // 2))
            else:
                prev = feats[level - 1]
                feats[level] = _resize(prev, ((prev.shape[1] + 1) // 2, (prev.shape[2] + 1) // 2))
        for i in range(cfg.num_layers):
            feats = getattr(self, f"layer{i}")(feats)
        return feats


class EfficientDetHead(BaseLayer):
    """Class and box towers of separable convolutions shared across levels; batch norms are per
    level.  Output format as ``RetinaNetHead``."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: int = 64
        num_classes: Required[int] = REQUIRED
        anchors_per_location: int = 9
        num_layers: int = 3
        min_level: int = 3
        max_level: int = 7
        prior_probability: float = 0.01

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        for tower in ("class", "box"):
            for i in range(cfg.num_layers):
                self._add_child(f"{tower}_conv{i}", SeparableConv.default_config().set(
                    input_dim=cfg.input_dim, output_dim=cfg.input_dim, norm=None))
                for level in range(cfg.min_level, cfg.max_level + 1):
                    self._add_child(f"{tower}_norm{i}_l{level}", BatchNorm.default_config().set(input_dim=cfg.input_dim))
        bias = -math.log((1 - cfg.prior_probability) / cfg.prior_probability)
        cls_init = DefaultInitializer.default_config().set(
            init_by_param_name={".*bias": ConstantInitializer.default_config().set(value=bias)})
        self._add_child("class_out", SeparableConv.default_config().set(
            input_dim=cfg.input_dim, output_dim=cfg.anchors_per_location * cfg.num_classes, norm=None,
            pointwise_param_init=cls_init))
        self._add_child("box_out", SeparableConv.default_config().set(
            input_dim=cfg.input_dim, output_dim=cfg.anchors_per_location * 4, norm=None))

    def forward(self, features: dict) -> dict:
        cfg = self._config
        cls_all, box_all = [], []
        for level in sorted(features):
            c = b = features[level]
            for i in range(cfg.num_layers):
                c = F.silu(getattr(self, f"class_norm{i}_l{level}")(getattr(self, f"class_conv{i}")(c)))
                b = F.silu(getattr(self, f"box_norm{i}_l{level}")(getattr(self, f"box_conv{i}")(b)))
            n = c.shape[0]
            cls_all.append(self.class_out(c).reshape(n, -1, cfg.num_classes))
            box_all.append(self.box_out(b).reshape(n, -1, 4))
        return {"class_outputs": torch.cat(cls_all, dim=1), "box_outputs": torch.cat(box_all, dim=1)}


# name: (backbone, BiFPN width, BiFPN layers, head layers, image size)
_SCALING = {
    "d0": ("efficientnet-b0", 64, 3, 3, 512), "d1": ("efficientnet-b1", 88, 4, 3, 640),
    "d2": ("efficientnet-b2", 112, 5, 3, 768), "d3": ("efficientnet-b3", 160, 6, 4, 896),
    "d4": ("efficientnet-b4", 224, 7, 4, 1024), "d5": ("efficientnet-b5", 288, 7, 4, 1280),
    "d6": ("efficientnet-b6", 384, 8, 5, 1280), "d7": ("efficientnet-b6", 384, 8, 5, 1536),
    "test": ("mobilenetv3-small-minimal-075", 16, 1, 1, 128),
}


def efficientdet_config(variant: str = "d0", *, num_classes: int = 90) -> InstantiableConfig:
    """``RetinaNetModel`` configured as EfficientDet-``variant`` (``d0`` ... ``d7``)."""
    backbone, width, fpn_layers, head_layers, _ = _SCALING[variant.lower()]
    cfg = RetinaNetModel.default_config().set(
        backbone=mobilenets.named_model_configs(backbone).set(embedding_dim=None), num_classes=num_classes,
        fpn=BiFPN.default_config().set(hidden_dim=width, num_layers=fpn_layers,
                                       fusion_method="fastattention" if variant.lower() != "d6" else "sum"),
        head=EfficientDetHead.default_config().set(num_layers=head_layers),
        anchor_size=4.0, box_loss_weight=50.0, focal_alpha=0.25, focal_gamma=1.5)
    return cfg


def image_size(variant: str) -> int:
    return _SCALING[variant.lower()][4]
