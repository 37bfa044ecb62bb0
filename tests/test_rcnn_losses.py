"""R-CNN stage losses against direct computations."""

import torch
import torch.nn.functional as F

from axlearn_b200.common.module import functional
from axlearn_b200.vision.rcnn_losses import RCNNDetectionMetric, RPNMetric


def _call(m, **kw):
    return functional(m, None, {}, kw, is_training=True)[0]


def _huber(err, delta):
    a = err.abs()
    return torch.where(a <= delta, 0.5 * a * a, delta * (a - 0.5 * delta))


def test_rpn_metric():
    torch.manual_seed(0)
    scores, boxes = torch.randn(2, 12), torch.randn(2, 12, 4)
    targets = (torch.rand(2, 12) > 0.6).float()
    box_targets = torch.randn(2, 12, 4)
    paddings = torch.rand(2, 12) > 0.7
    m = RPNMetric.default_config().set(name="m", box_loss_weight=2.0).instantiate(parent=None)
    got = _call(m, outputs={"rpn_scores": scores, "rpn_boxes": boxes},
            labels={"rpn_score_targets": targets, "rpn_box_targets": box_targets}, paddings=paddings)
    live = ~paddings
    want_score = (F.binary_cross_entropy_with_logits(scores, targets, reduction="none") * live).sum() / live.sum()
    pos = live & (targets > 0)
    want_box = (_huber(boxes - box_targets, 1 / 9).mean(-1) * pos).sum() / pos.sum()
    torch.testing.assert_close(got, want_score + 2.0 * want_box, atol=1e-5, rtol=1e-5)
    # Everything padded: finite, zero.
    zero = _call(m, outputs={"rpn_scores": scores, "rpn_boxes": boxes},
             labels={"rpn_score_targets": targets, "rpn_box_targets": box_targets}, paddings=torch.ones_like(paddings))
    assert zero.item() == 0.0


def test_rcnn_detection_metric_shared_and_per_class_boxes():
    torch.manual_seed(1)
    num_classes = 4
    logits = torch.randn(2, 6, num_classes)
    targets = torch.tensor([[0, 1, 3, 2, 0, 1], [2, 0, 0, 3, 1, 1]])
    box_targets = torch.randn(2, 6, 4)
    paddings = torch.tensor([[False] * 5 + [True], [False] * 4 + [True] * 2])
    live = ~paddings
    want_cls = (F.cross_entropy(logits.reshape(-1, num_classes), targets.reshape(-1), reduction="none").reshape(2, 6) * live).sum() / live.sum()
    pos = live & (targets > 0)
    m = RCNNDetectionMetric.default_config().set(name="m", num_classes=num_classes).instantiate(parent=None)
    shared = torch.randn(2, 6, 4)
    got = _call(m, outputs={"class_scores": logits, "boxes": shared}, labels={"class_targets": targets, "box_targets": box_targets},
            paddings=paddings)
    want_box = (_huber(shared - box_targets, 1.0).mean(-1) * pos).sum() / pos.sum()
    torch.testing.assert_close(got, want_cls + want_box, atol=1e-5, rtol=1e-5)
    per_class = torch.randn(2, 6, num_classes * 4)
    got = _call(m, outputs={"class_scores": logits, "boxes": per_class}, labels={"class_targets": targets, "box_targets": box_targets},
            paddings=paddings)
    chosen = per_class.reshape(2, 6, num_classes, 4)[torch.arange(2)[:, None], torch.arange(6)[None], targets]
    want_box = (_huber(chosen - box_targets, 1.0).mean(-1) * pos).sum() / pos.sum()
    torch.testing.assert_close(got, want_cls + want_box, atol=1e-5, rtol=1e-5)
