"""Feature pyramid network and RetinaNet (one-stage detector with focal loss).

Parity targets in the reference: axlearn/vision/fpn.py (``FPN`` :60: lateral 1x1 convolutions,
top-down nearest upsampling and sum, 3x3 output convolutions, extra coarser levels by stride-2
convolutions), axlearn/vision/retinanet.py (``RetinaNetHead`` :40: per-level class and box towers
of ``num_layers`` 3x3 convolutions shared across levels with per-level norms, class bias
initialised to ``-log((1 - pi) / pi)``; ``RetinaNetMetric`` :180: sigmoid focal loss + Huber box
loss normalised by the number of positive anchors; ``RetinaNetModel`` :300),
axlearn/vision/matchers.py / anchor labeling (positives IoU >= 0.5, negatives < 0.4, the rest
ignored) and axlearn/vision/detection_generator.py (decode boxes, per-class NMS).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.param_init import ConstantInitializer, DefaultInitializer
from axlearn_b200.vision import detection_utils as det

Tensor = torch.Tensor


def _conv(window: int, stride: int = 1) -> Conv2D.Config:
    return Conv2D.default_config().set(window=(window, window), strides=(stride, stride), padding="SAME", bias=True)


def _upsample_nearest(x: Tensor, size) -> Tensor:
    """``[B, h, w, C] -> [B, H, W, C]`` nearest-neighbour (index gather: works for any ratio)."""
    h, w = x.shape[1:3]
    rows = (torch.arange(size[0], device=x.device) * h) // size[0]
    cols = (torch.arange(size[1], device=x.device) * w) // size[1]
    return x[:, rows][:, :, cols]


class FPN(BaseLayer):
    """``{level: [B, H_l, W_l, C_l]}`` for the backbone levels -> ``{level: [B, H_l, W_l, hidden_dim]}``
    for ``min_level .. max_level`` (levels above the backbone's coarsest are made by stride-2
    convolutions of the level below)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dims: Required[dict] = REQUIRED          # {"3": 512, "4": 1024, "5": 2048}
        hidden_dim: int = 256
        min_level: int = 3
        max_level: int = 7

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._backbone_levels = sorted(int(k) for k in cfg.input_dims if min(cfg.min_level, 2) <= int(k) <= cfg.max_level
                                       and int(k) >= cfg.min_level)
        for level in self._backbone_levels:
            self._add_child(f"lateral{level}", _conv(1).set(input_dim=cfg.input_dims[str(level)], output_dim=cfg.hidden_dim))
            self._add_child(f"output{level}", _conv(3).set(input_dim=cfg.hidden_dim, output_dim=cfg.hidden_dim))
        for level in range(self._backbone_levels[-1] + 1, cfg.max_level + 1):
            self._add_child(f"coarse{level}", _conv(3, 2).set(input_dim=cfg.hidden_dim, output_dim=cfg.hidden_dim))

    def forward(self, endpoints: dict) -> dict:
        cfg = self._config
        levels = self._backbone_levels
        feats = {l: getattr(self, f"lateral{l}")(endpoints[str(l)]) for l in levels}
        for l in reversed(levels[:-1]):
            feats[l] = feats[l] + _upsample_nearest(feats[l + 1], feats[l].shape[1:3])
        out = {l: getattr(self, f"output{l}")(feats[l]) for l in levels}
        for l in range(levels[-1] + 1, cfg.max_level + 1):
            x = out[l - 1]
            out[l] = getattr(self, f"coarse{l}")(F.relu(x) if l > levels[-1] + 1 else x)
        return out


class RetinaNetHead(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: int = 256
        num_classes: Required[int] = REQUIRED
        anchors_per_location: int = 9
        num_layers: int = 4
        prior_probability: float = 0.01

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        for tower in ("class", "box"):
            for i in range(cfg.num_layers):
                self._add_child(f"{tower}_conv{i}", _conv(3).set(input_dim=cfg.input_dim, output_dim=cfg.input_dim))
        bias = -math.log((1 - cfg.prior_probability) / cfg.prior_probability)
        cls_init = DefaultInitializer.default_config().set(
            init_by_param_name={".*bias": ConstantInitializer.default_config().set(value=bias)})
        self._add_child("class_out", _conv(3).set(input_dim=cfg.input_dim,
                                                  output_dim=cfg.anchors_per_location * cfg.num_classes, param_init=cls_init))
        self._add_child("box_out", _conv(3).set(input_dim=cfg.input_dim, output_dim=cfg.anchors_per_location * 4))

    def forward(self, features: dict) -> dict:
        """``{"class_outputs": [B, A_total, num_classes], "box_outputs": [B, A_total, 4]}``, anchors
        ordered by level, then row-major cells, then anchor index -- the order of
        ``generate_anchors``."""
        cfg = self._config
        cls_all, box_all = [], []
        for level in sorted(features):
            c = b = features[level]
            for i in range(cfg.num_layers):
                c = F.relu(getattr(self, f"class_conv{i}")(c))
                b = F.relu(getattr(self, f"box_conv{i}")(b))
            n = c.shape[0]
            cls_all.append(self.class_out(c).reshape(n, -1, cfg.num_classes))
            box_all.append(self.box_out(b).reshape(n, -1, 4))
        return {"class_outputs": torch.cat(cls_all, dim=1), "box_outputs": torch.cat(box_all, dim=1)}


def label_anchors(anchors: Tensor, gt_boxes: Tensor, gt_classes: Tensor, *, foreground_iou: float = 0.5,
                  background_iou: float = 0.4) -> tuple[Tensor, Tensor, Tensor]:
    """One image: ``anchors [A, 4]``, ``gt_boxes [G, 4]``, ``gt_classes [G]`` (< 0 = padding) ->
    (class targets ``[A]``: class id, -1 background, -2 ignore; box targets ``[A, 4]`` = the
    matched ground-truth box; positive mask ``[A]``)."""
    valid = gt_classes >= 0
    if not valid.any():
        a = anchors.shape[0]
        return torch.full((a,), -1, dtype=torch.long), torch.zeros(a, 4), torch.zeros(a, dtype=torch.bool)
    iou = det.pairwise_iou(anchors, gt_boxes)
    iou = torch.where(valid[None], iou, torch.full_like(iou, -1.0))
    best_iou, best_gt = iou.max(dim=1)
    cls = torch.full_like(best_gt, -2)
    cls[best_iou < background_iou] = -1
    positive = best_iou >= foreground_iou
    cls[positive] = gt_classes[best_gt[positive]].long()
    return cls, gt_boxes[best_gt], positive


def sigmoid_focal_loss(logits: Tensor, targets: Tensor, *, alpha: float = 0.25, gamma: float = 1.5) -> Tensor:
    """Element-wise focal loss; ``targets`` in {0, 1}."""
    p = torch.sigmoid(logits)
    ce = F.binary_cross_entropy_with_logits(logits, targets, reduction="none")
    p_t = p * targets + (1 - p) * (1 - targets)
    a_t = alpha * targets + (1 - alpha) * (1 - targets)
    return a_t * (1 - p_t) ** gamma * ce


class RetinaNetModel(BaseModel):
    """``input_batch = {"image": [B, H, W, 3], "groundtruth_boxes": [B, G, 4], "groundtruth_classes":
    [B, G]}`` (classes < 0 pad)."""

    @config_class
    class Config(BaseModel.Config):
        backbone: Required[InstantiableConfig] = REQUIRED
        fpn: InstantiableConfig = FPN.default_config()
        head: InstantiableConfig = RetinaNetHead.default_config()
        num_classes: Required[int] = REQUIRED
        num_scales: int = 3
        aspect_ratios: Sequence[float] = (1.0, 2.0, 0.5)
        anchor_size: float = 4.0
        box_loss_weight: float = 50.0
        huber_delta: float = 0.1
        focal_alpha: float = 0.25
        focal_gamma: float = 1.5
        box_coder_weights: Sequence[float] = (1.0, 1.0, 1.0, 1.0)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("backbone", cfg.backbone)
        dims = {k: v for k, v in self.backbone.endpoints_dims.items() if k.isdigit()}
        self._add_child("fpn", cfg.fpn.clone(input_dims=dims))
        self._add_child("head", cfg.head.clone(
            input_dim=cfg.fpn.hidden_dim, num_classes=cfg.num_classes,
            anchors_per_location=cfg.num_scales * len(cfg.aspect_ratios)))

    def _anchors(self, image_shape) -> Tensor:
        cfg = self._config
        per_level = det.generate_anchors(
            image_shape=image_shape, min_level=cfg.fpn.min_level, max_level=cfg.fpn.max_level,
            num_scales=cfg.num_scales, aspect_ratios=cfg.aspect_ratios, anchor_size=cfg.anchor_size)
        return torch.cat([per_level[l] for l in sorted(per_level)], dim=0)

    def predict(self, input_batch: dict) -> dict:
        image = input_batch["image"]
        out = self.head(self.fpn(self.backbone(image)))
        out["anchors"] = self._anchors(image.shape[1:3]).to(image.device)
        return out

    def forward(self, input_batch: dict):
        cfg = self._config
        out = self.predict(input_batch)
        anchors = out["anchors"]
        cls_logits, box_out = out["class_outputs"].float(), out["box_outputs"].float()
        b = cls_logits.shape[0]
        cls_loss = box_loss = cls_logits.new_zeros(())
        num_pos = cls_logits.new_zeros(())
        for i in range(b):
            cls_t, box_t, pos = label_anchors(anchors, input_batch["groundtruth_boxes"][i].float(),
                                              input_batch["groundtruth_classes"][i])
            keep = cls_t != -2
            one_hot = F.one_hot(cls_t.clamp_min(0), cfg.num_classes).float() * (cls_t >= 0)[:, None]
            fl = sigmoid_focal_loss(cls_logits[i], one_hot, alpha=cfg.focal_alpha, gamma=cfg.focal_gamma)
            cls_loss = cls_loss + (fl * keep[:, None]).sum()
            if pos.any():
                target = det.encode_boxes(box_t[pos], anchors[pos], cfg.box_coder_weights)
                box_loss = box_loss + F.huber_loss(box_out[i][pos], target, delta=cfg.huber_delta, reduction="sum")
            num_pos = num_pos + pos.sum()
        norm = num_pos.clamp_min(1.0)
        cls_loss, box_loss = cls_loss / norm, box_loss / norm
        loss = cls_loss + cfg.box_loss_weight * box_loss
        self.add_summary("loss/class", WeightedSummary(cls_loss.detach(), norm))
        self.add_summary("loss/box", WeightedSummary(box_loss.detach(), norm))
        self.add_summary("num_positive_anchors", num_pos / b)
        return loss, out

    def detect(self, input_batch: dict, *, score_threshold: float = 0.05, iou_threshold: float = 0.5,
               max_detections: int = 100) -> list[dict]:
        """Per image: ``{"boxes" [N, 4], "scores" [N], "classes" [N]}`` after decoding, clipping and
        per-class NMS."""
        cfg = self._config
        out = self.predict(input_batch)
        shape = input_batch["image"].shape[1:3]
        results = []
        for cls_logits, deltas in zip(out["class_outputs"], out["box_outputs"]):
            boxes = det.clip_boxes(det.decode_boxes(deltas.float(), out["anchors"], cfg.box_coder_weights), shape)
            scores = torch.sigmoid(cls_logits.float())
            found = []
            for c in range(cfg.num_classes):
                idx, valid = det.non_max_suppression(boxes, scores[:, c], iou_threshold=iou_threshold,
                                                     max_output_size=max_detections, score_threshold=score_threshold)
                for j in idx[valid].tolist():
                    found.append((scores[j, c].item(), c, boxes[j]))
            found.sort(key=lambda t: -t[0])
            found = found[:max_detections]
            results.append({
                "boxes": torch.stack([f[2] for f in found]) if found else torch.zeros(0, 4),
                "scores": torch.tensor([f[0] for f in found]), "classes": torch.tensor([f[1] for f in found], dtype=torch.long)})
        return results
