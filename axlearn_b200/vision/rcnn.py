"""Two-stage detection: region proposal network, ROI sampling and alignment, box head, Faster R-CNN.

Reference: axlearn/vision/rcnn.py (``FasterRCNN`` :33-307), detection_heads.py (``RPNHead``,
``RCNNDetectionHead``), roi_generator.py, rpn_sampler.py, rcnn_sampler.py, roi_aligner.py
(multi-level ROI align), rcnn_losses.py and detection_generator.py (per-class NMS).

Pipeline per image: backbone -> FPN levels 2..6 -> RPN objectness / deltas per anchor -> top-k
decode + NMS -> proposals; in training a subset of anchors trains the RPN (objectness BCE + Huber
on deltas) and a fixed-size sample of proposals (25 % foreground by IoU >= 0.5, plus the ground
truth boxes) trains the box head (softmax CE + Huber on class-agnostic deltas); every ROI is
pooled from the pyramid level ``floor(4 + log2(sqrt(area) / 224))``.  Boxes are ``(y0, x0, y1,
x1)`` in pixels; padded ground-truth rows have class < 0.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from axlearn_b200.common import prng
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.convolution import Conv2D
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.vision import detection_utils as det
from axlearn_b200.vision.retinanet import FPN

Tensor = torch.Tensor


def _conv(window: int) -> InstantiableConfig:
    pad = (window - 1) // 2
    return Conv2D.default_config().set(window=(window, window), padding=((pad, pad), (pad, pad)), bias=True)


class RPNHead(BaseLayer):
    """A shared 3x3 convolution, then per anchor one objectness logit and four box deltas."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        anchors_per_location: int = 3

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("conv", _conv(3).set(input_dim=cfg.input_dim, output_dim=cfg.input_dim))
        self._add_child("scores", _conv(1).set(input_dim=cfg.input_dim, output_dim=cfg.anchors_per_location))
        self._add_child("boxes", _conv(1).set(input_dim=cfg.input_dim, output_dim=4 * cfg.anchors_per_location))

    def forward(self, features: dict) -> tuple[Tensor, Tensor]:
        """``{level: [B, H, W, C]}`` -> scores ``[B, A_total]`` and deltas ``[B, A_total, 4]`` in the
        anchor order of ``generate_anchors`` (levels ascending, row-major cells, anchors last)."""
        scores, boxes = [], []
        for level in sorted(features):
            h = F.relu(self.conv(features[level]))
            b = h.shape[0]
            scores.append(self.scores(h).reshape(b, -1))
            boxes.append(self.boxes(h).reshape(b, -1, 4))
        return torch.cat(scores, dim=1), torch.cat(boxes, dim=1)


def generate_proposals(*, scores: Tensor, deltas: Tensor, anchors: Tensor, image_shape: Sequence[int],
                       pre_nms_top_k: int = 1000, post_nms_top_k: int = 300, nms_iou: float = 0.7,
                       min_size: float = 0.0) -> tuple[Tensor, Tensor]:
    """One image: the ``pre_nms_top_k`` best anchors are decoded, clipped and reduced by NMS to
    ``[post_nms_top_k, 4]`` proposals with a validity mask."""
    k = min(pre_nms_top_k, scores.shape[0])
    top, idx = scores.topk(k)
    boxes = det.clip_boxes(det.decode_boxes(deltas[idx], anchors[idx]), image_shape)
    hw = boxes[:, 2:] - boxes[:, :2]
    ok = (hw > min_size).all(dim=-1)
    top = torch.where(ok, top, torch.full_like(top, -1e9))
    keep, valid = det.non_max_suppression(boxes, top, iou_threshold=nms_iou, max_output_size=post_nms_top_k,
                                          score_threshold=-1e8)
    return boxes[keep.clamp_min(0)] * valid[:, None], valid


def _sample(mask_pos: Tensor, mask_neg: Tensor, *, size: int, positive_fraction: float, key) -> tuple[Tensor, Tensor]:
    """Picks up to ``size * positive_fraction`` positives and fills with negatives (random subsets).
    Returns index ``[size]`` and validity ``[size]``."""
    n = mask_pos.shape[0]
    noise = prng.uniform(key, (n,)) if key is not None else torch.linspace(0.9, 0.1, n)
    pos_rank = torch.argsort(torch.where(mask_pos, noise, torch.full_like(noise, -1.0)), descending=True)
    neg_rank = torch.argsort(torch.where(mask_neg, noise, torch.full_like(noise, -1.0)), descending=True)
    num_pos = min(int(mask_pos.sum()), int(size * positive_fraction))
    num_neg = min(int(mask_neg.sum()), size - num_pos)
    idx = torch.cat([pos_rank[:num_pos], neg_rank[:num_neg]])
    valid = torch.ones(idx.shape[0], dtype=torch.bool)
    pad = size - idx.shape[0]
    if pad:
        idx = torch.cat([idx, torch.zeros(pad, dtype=idx.dtype)])
        valid = torch.cat([valid, torch.zeros(pad, dtype=torch.bool)])
    return idx, valid


def roi_levels(boxes: Tensor, *, min_level: int, max_level: int, canonical_level: int = 4,
               canonical_size: float = 224.0) -> Tensor:
    area = ((boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1])).clamp_min(1e-6)
    level = torch.floor(canonical_level + torch.log2(torch.sqrt(area) / canonical_size))
    return level.clamp(min_level, max_level).long()


def multilevel_roi_align(features: dict, boxes: Tensor, *, output_size: int = 7) -> Tensor:
    """One image: ``{level: [H, W, C]}``, ``boxes [N, 4]`` in pixels -> ``[N, s, s, C]``."""
    levels = sorted(features)
    assigned = roi_levels(boxes, min_level=levels[0], max_level=levels[-1])
    c = features[levels[0]].shape[-1]
    out = boxes.new_zeros(boxes.shape[0], output_size, output_size, c, dtype=features[levels[0]].dtype)
    for level in levels:
        sel = (assigned == level).nonzero().squeeze(-1)
        if sel.numel():
            out[sel] = det.roi_align(features[level], boxes[sel] / 2 ** level, output_size=output_size)
    return out


class RCNNDetectionHead(BaseLayer):
    """Pooled ROI features -> fully connected layers -> class logits and class-agnostic deltas."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        roi_size: int = 7
        num_classes: Required[int] = REQUIRED          # foreground classes; class 0 of the logits is background
        hidden_dim: int = 1024
        num_fc_layers: int = 2

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        dim = cfg.input_dim * cfg.roi_size ** 2
        for i in range(cfg.num_fc_layers):
            self._add_child(f"fc{i}", Linear.default_config().set(input_dim=dim, output_dim=cfg.hidden_dim))
            dim = cfg.hidden_dim
        self._add_child("classes", Linear.default_config().set(input_dim=dim, output_dim=cfg.num_classes + 1))
        self._add_child("boxes", Linear.default_config().set(input_dim=dim, output_dim=4))

    def forward(self, rois: Tensor) -> tuple[Tensor, Tensor]:
        x = rois.reshape(rois.shape[0], -1)
        for i in range(self._config.num_fc_layers):
            x = F.relu(getattr(self, f"fc{i}")(x))
        return self.classes(x), self.boxes(x)


class FasterRCNN(BaseModel):
    """``input_batch``: ``image [B, H, W, 3]``, ``gt_boxes [B, G, 4]``, ``gt_classes [B, G]``
    (1-based foreground classes; < 0 = padding)."""

    @config_class
    class Config(BaseModel.Config):
        backbone: Required[InstantiableConfig] = REQUIRED
        num_classes: Required[int] = REQUIRED
        fpn: InstantiableConfig = FPN.default_config().set(min_level=2, max_level=6)
        rpn_head: InstantiableConfig = RPNHead.default_config()
        rcnn_head: InstantiableConfig = RCNNDetectionHead.default_config()
        anchor_size: float = 8.0
        aspect_ratios: Sequence[float] = (1.0, 2.0, 0.5)
        rpn_batch_size: int = 256
        rpn_positive_fraction: float = 0.5
        rpn_foreground_iou: float = 0.7
        rpn_background_iou: float = 0.3
        pre_nms_top_k: int = 1000
        post_nms_top_k: int = 300
        rpn_nms_iou: float = 0.7
        roi_batch_size: int = 128
        roi_positive_fraction: float = 0.25
        roi_foreground_iou: float = 0.5
        box_weights: Sequence[float] = (10.0, 10.0, 5.0, 5.0)
        huber_delta: float = 1.0 / 9.0
        detection_score_threshold: float = 0.05
        detection_nms_iou: float = 0.5
        max_detections: int = 100

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("backbone", cfg.backbone)
        dims = self.backbone.endpoints_dims
        fpn = cfg.fpn.clone(input_dims={k: v for k, v in dims.items() if k.isdigit()})
        self._add_child("fpn", fpn)
        self._add_child("rpn_head", cfg.rpn_head.clone(input_dim=fpn.hidden_dim, anchors_per_location=len(cfg.aspect_ratios)))
        self._add_child("rcnn_head", cfg.rcnn_head.clone(input_dim=fpn.hidden_dim, num_classes=cfg.num_classes))

    # ---------------------------------------------------------------- shared
    def _anchors(self, image_shape) -> Tensor:
        cfg = self._config
        per_level = det.generate_anchors(image_shape=image_shape, min_level=cfg.fpn.min_level, max_level=cfg.fpn.max_level,
                                         num_scales=1, aspect_ratios=cfg.aspect_ratios, anchor_size=cfg.anchor_size)
        return torch.cat([per_level[l] for l in sorted(per_level)], dim=0)

    def _first_stage(self, image: Tensor):
        cfg = self._config
        features = self.fpn(self.backbone(image))
        scores, deltas = self.rpn_head(features)
        anchors = self._anchors(image.shape[1:3]).to(image.device)
        proposals, valid = [], []
        for b in range(image.shape[0]):
            p, v = generate_proposals(scores=scores[b].detach().float(), deltas=deltas[b].detach().float(), anchors=anchors,
                                      image_shape=image.shape[1:3], pre_nms_top_k=cfg.pre_nms_top_k,
                                      post_nms_top_k=cfg.post_nms_top_k, nms_iou=cfg.rpn_nms_iou)
            proposals.append(p)
            valid.append(v)
        return features, scores, deltas, anchors, torch.stack(proposals), torch.stack(valid)

    def _huber(self, pred: Tensor, target: Tensor) -> Tensor:
        d = self._config.huber_delta
        err = (pred - target).abs()
        return torch.where(err < d, 0.5 * err ** 2 / d, err - 0.5 * d).sum(-1)

    # ---------------------------------------------------------------- training
    def forward(self, input_batch: dict):
        cfg = self._config
        image, gt_boxes, gt_classes = input_batch["image"], input_batch["gt_boxes"].float(), input_batch["gt_classes"]
        features, scores, deltas, anchors, proposals, proposal_valid = self._first_stage(image)
        keys = prng.split(self.prng_key, 2 * image.shape[0]) if self.is_training else [None] * (2 * image.shape[0])
        rpn_cls, rpn_box, rcnn_cls, rcnn_box = [], [], [], []
        for b in range(image.shape[0]):
            live_gt = gt_classes[b] >= 0
            # RPN targets.
            iou = det.pairwise_iou(anchors, gt_boxes[b])
            iou = torch.where(live_gt[None], iou, torch.full_like(iou, -1.0))
            best, match = iou.max(dim=1) if live_gt.any() else (torch.full((anchors.shape[0],), -1.0), torch.zeros(anchors.shape[0], dtype=torch.long))
            pos, neg = best >= cfg.rpn_foreground_iou, (best < cfg.rpn_background_iou)
            if live_gt.any():                      # every ground-truth box keeps its best anchor
                pos = pos | (iou == iou.max(dim=0).values[None]).any(dim=1) & (best > 0)
            idx, ok = _sample(pos, neg & ~pos, size=cfg.rpn_batch_size, positive_fraction=cfg.rpn_positive_fraction, key=keys[2 * b])
            target = pos[idx].float()
            n = ok.sum().clamp_min(1)
            rpn_cls.append((F.binary_cross_entropy_with_logits(scores[b, idx].float(), target, reduction="none") * ok).sum() / n)
            enc = det.encode_boxes(gt_boxes[b][match[idx]], anchors[idx])
            rpn_box.append((self._huber(deltas[b, idx].float(), enc) * (ok & pos[idx])).sum() / n)
            # Box-head targets: proposals plus the ground truth, matched by IoU.
            rois = torch.cat([proposals[b][proposal_valid[b]], gt_boxes[b][live_gt]], dim=0)
            if rois.shape[0] == 0:
                continue
            r_iou = det.pairwise_iou(rois, gt_boxes[b])
            r_iou = torch.where(live_gt[None], r_iou, torch.full_like(r_iou, -1.0))
            r_best, r_match = r_iou.max(dim=1)
            fg = r_best >= cfg.roi_foreground_iou
            ridx, rok = _sample(fg, ~fg, size=cfg.roi_batch_size, positive_fraction=cfg.roi_positive_fraction, key=keys[2 * b + 1])
            sampled = rois[ridx]
            labels = torch.where(fg[ridx], gt_classes[b][r_match[ridx]].long(), torch.zeros_like(ridx))
            pooled = multilevel_roi_align({l: f[b] for l, f in features.items()}, sampled, output_size=cfg.rcnn_head.roi_size)
            logits, box = self.rcnn_head(pooled)
            m = rok.sum().clamp_min(1)
            rcnn_cls.append((F.cross_entropy(logits.float(), labels, reduction="none") * rok).sum() / m)
            enc = det.encode_boxes(gt_boxes[b][r_match[ridx]], sampled, weights=cfg.box_weights)
            rcnn_box.append((self._huber(box.float(), enc) * (rok & fg[ridx])).sum() / m)
        mean = lambda xs: torch.stack(xs).mean() if xs else scores.sum() * 0
        losses = dict(rpn_score_loss=mean(rpn_cls), rpn_box_loss=mean(rpn_box), frcnn_class_loss=mean(rcnn_cls),
                      frcnn_box_loss=mean(rcnn_box))
        for k, v in losses.items():
            self.add_summary(k, WeightedSummary(v.detach(), image.shape[0]))
        return sum(losses.values()), losses

    # ---------------------------------------------------------------- inference
    @torch.no_grad()
    def predict(self, input_batch: dict) -> dict:
        """``detection_boxes [B, D, 4]``, ``detection_scores``, ``detection_classes`` (1-based),
        ``num_detections``; per-class NMS over the refined proposals."""
        cfg = self._config
        image = input_batch["image"]
        features, _, _, _, proposals, proposal_valid = self._first_stage(image)
        d = cfg.max_detections
        out = dict(detection_boxes=image.new_zeros(image.shape[0], d, 4), detection_scores=image.new_zeros(image.shape[0], d),
                   detection_classes=torch.zeros(image.shape[0], d, dtype=torch.long),
                   num_detections=torch.zeros(image.shape[0], dtype=torch.long))
        for b in range(image.shape[0]):
            rois = proposals[b][proposal_valid[b]]
            if rois.shape[0] == 0:
                continue
            pooled = multilevel_roi_align({l: f[b] for l, f in features.items()}, rois, output_size=cfg.rcnn_head.roi_size)
            logits, box = self.rcnn_head(pooled)
            probs = torch.softmax(logits.float(), dim=-1)[:, 1:]
            boxes = det.clip_boxes(det.decode_boxes(box.float(), rois, weights=cfg.box_weights), image.shape[1:3])
            cand_boxes, cand_scores, cand_classes = [], [], []
            for c in range(probs.shape[1]):
                keep, valid = det.non_max_suppression(boxes, probs[:, c], iou_threshold=cfg.detection_nms_iou,
                                                      max_output_size=d, score_threshold=cfg.detection_score_threshold)
                keep = keep[valid]
                cand_boxes.append(boxes[keep])
                cand_scores.append(probs[keep, c])
                cand_classes.append(torch.full((keep.shape[0],), c + 1, dtype=torch.long))
            cb, cs, cc = torch.cat(cand_boxes), torch.cat(cand_scores), torch.cat(cand_classes)
            top = torch.argsort(cs, descending=True)[:d]
            n = top.shape[0]
            out["detection_boxes"][b, :n], out["detection_scores"][b, :n] = cb[top], cs[top]
            out["detection_classes"][b, :n], out["num_detections"][b] = cc[top], n
        return out
