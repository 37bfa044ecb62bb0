"""Encoding of boxes relative to anchors (reference: axlearn/vision/box_coder.py:15-162; the Faster
R-CNN parameterisation, arXiv:1506.01497): ``(dy, dx)`` are centre offsets in units of the anchor's
size, ``(dh, dw)`` log size ratios, each multiplied by a weight."""

from __future__ import annotations

import enum
import math

import torch

from axlearn_b200.common.config import Configurable, config_class

Tensor = torch.Tensor

BBOX_XFORM_CLIP_EXP = 1000.0 / 16.0
BBOX_XFORM_CLIP = math.log(BBOX_XFORM_CLIP_EXP)


class BoxClipMethod(str, enum.Enum):
    """How decoded offsets are limited: not at all; height / width offsets from above (so that
    ``exp`` cannot overflow); or all four offsets from both sides."""

    NONE = "None"
    MaxHW = "MaxHW"
    MinMaxYXHW = "MinMaxYXHW"


class BoxCoder(Configurable):
    @config_class
    class Config(Configurable.Config):
        eps: float = 1e-8
        box_wh_min_value: float = 0.0
        weights: tuple = (1.0, 1.0, 1.0, 1.0)
        clip_boxes: BoxClipMethod = BoxClipMethod.MaxHW

    def encode(self, *, boxes: Tensor, anchors: Tensor) -> Tensor:
        """``boxes`` and ``anchors`` ``[..., 4]`` as ``[ymin, xmin, ymax, xmax]`` (anchors broadcast)."""
        cfg = self._config
        boxes = boxes.to(anchors.dtype)
        box_h = (boxes[..., 2] - boxes[..., 0] + cfg.eps).clamp(min=cfg.box_wh_min_value)
        box_w = (boxes[..., 3] - boxes[..., 1] + cfg.eps).clamp(min=cfg.box_wh_min_value)
        box_yc, box_xc = boxes[..., 0] + 0.5 * box_h, boxes[..., 1] + 0.5 * box_w
        anchor_h = anchors[..., 2] - anchors[..., 0] + cfg.eps
        anchor_w = anchors[..., 3] - anchors[..., 1] + cfg.eps
        anchor_yc, anchor_xc = anchors[..., 0] + 0.5 * anchor_h, anchors[..., 1] + 0.5 * anchor_w
        w = cfg.weights
        return torch.stack([(box_yc - anchor_yc) / anchor_h * w[0], (box_xc - anchor_xc) / anchor_w * w[1],
                            torch.log(box_h / anchor_h) * w[2], torch.log(box_w / anchor_w) * w[3]], dim=-1)

    def decode(self, *, encoded_boxes: Tensor, anchors: Tensor) -> Tensor:
        cfg = self._config
        e = encoded_boxes.to(anchors.dtype)
        w = cfg.weights
        dy, dx, dh, dw = e[..., 0] / w[0], e[..., 1] / w[1], e[..., 2] / w[2], e[..., 3] / w[3]
        if cfg.clip_boxes == BoxClipMethod.MaxHW:
            dh, dw = dh.clamp(max=BBOX_XFORM_CLIP), dw.clamp(max=BBOX_XFORM_CLIP)
        elif cfg.clip_boxes == BoxClipMethod.MinMaxYXHW:
            dy, dx = dy.clamp(-BBOX_XFORM_CLIP_EXP, BBOX_XFORM_CLIP_EXP), dx.clamp(-BBOX_XFORM_CLIP_EXP, BBOX_XFORM_CLIP_EXP)
            dh, dw = dh.clamp(-BBOX_XFORM_CLIP, BBOX_XFORM_CLIP), dw.clamp(-BBOX_XFORM_CLIP, BBOX_XFORM_CLIP)
        anchor_h, anchor_w = anchors[..., 2] - anchors[..., 0], anchors[..., 3] - anchors[..., 1]
        yc = dy * anchor_h + anchors[..., 0] + 0.5 * anchor_h
        xc = dx * anchor_w + anchors[..., 1] + 0.5 * anchor_w
        h, w_ = torch.exp(dh) * anchor_h, torch.exp(dw) * anchor_w
        ymin, xmin = yc - 0.5 * h, xc - 0.5 * w_
        return torch.stack([ymin, xmin, ymin + h, xmin + w_], dim=-1)
