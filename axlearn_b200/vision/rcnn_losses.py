"""Losses of the two Faster R-CNN stages (reference: axlearn/vision/rcnn_losses.py:17-173)."""

from __future__ import annotations

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.loss import ReductionMethod, cross_entropy, huber_loss, sigmoid_cross_entropy_with_logits

Tensor = torch.Tensor


class RPNMetric(BaseLayer):
    """Binary cross entropy on proposal scores (mean over sampled anchors) plus Huber loss on the
    box encodings of the positive ones (mean over positives, coordinates averaged)."""

    @config_class
    class Config(BaseLayer.Config):
        huber_loss_delta: float = 1.0 / 9.0
        box_loss_weight: float = 1.0
        score_loss_weight: float = 1.0
        normalizer_eps: float = 1e-08

    def forward(self, *, outputs: dict, labels: dict, paddings: Tensor) -> Tensor:
        """``outputs``: ``rpn_scores [..., P]`` (logits), ``rpn_boxes [..., P, 4]``; ``labels``:
        ``rpn_score_targets`` in {0, 1}, ``rpn_box_targets``; ``paddings [..., P]`` bool."""
        cfg = self._config
        live = ~paddings.bool()
        true_scores = labels["rpn_score_targets"]
        score_loss = (sigmoid_cross_entropy_with_logits(outputs["rpn_scores"], true_scores) * live).sum() / (
            live.sum() + cfg.normalizer_eps)
        box_weights = live & (true_scores > 0)
        box_loss = huber_loss(predictions=outputs["rpn_boxes"], targets=labels["rpn_box_targets"],
                              delta=cfg.huber_loss_delta, reduce_axis=-1,
                              sample_weight=box_weights / (box_weights.sum() + cfg.normalizer_eps),
                              reduction=ReductionMethod.SUM)
        return cfg.score_loss_weight * score_loss + cfg.box_loss_weight * box_loss


class RCNNDetectionMetric(BaseLayer):
    """Softmax cross entropy over ``num_classes`` (0 = background) plus Huber loss on the box
    encodings of foreground detections.  With per-class box outputs (``boxes [..., P, C * 4]``) the
    box predicted for the target class is the one that is trained; ``C = 1`` shares one box."""

    @config_class
    class Config(BaseLayer.Config):
        huber_loss_delta: float = 1.0
        box_loss_weight: float = 1.0
        class_loss_weight: float = 1.0
        num_classes: Required[int] = REQUIRED
        normalizer_eps: float = 1e-08

    def forward(self, *, outputs: dict, labels: dict, paddings: Tensor) -> Tensor:
        cfg = self._config
        live = ~paddings.bool()
        targets = labels["class_targets"]
        _, aux = cross_entropy(outputs["class_scores"], targets.clamp(min=0), live_targets=live)
        score_loss = aux["cross_entropy_loss"]
        box_weights = live & (targets > 0)
        pred = outputs["boxes"]
        batch, num_boxes, num_coordinates = pred.shape
        classes_for_boxes = num_coordinates // 4
        pred = pred.reshape(batch, num_boxes, classes_for_boxes, 4)
        ids = targets.clamp(min=0, max=classes_for_boxes - 1)
        pred = torch.gather(pred, 2, ids[..., None, None].expand(-1, -1, 1, 4))[..., 0, :]
        box_loss = huber_loss(predictions=pred, targets=labels["box_targets"], delta=cfg.huber_loss_delta, reduce_axis=-1,
                              sample_weight=box_weights / (box_weights.sum() + cfg.normalizer_eps),
                              reduction=ReductionMethod.SUM)
        return cfg.class_loss_weight * score_loss + cfg.box_loss_weight * box_loss
