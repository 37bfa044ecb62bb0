"""Faster R-CNN pieces and an overfitting run on one synthetic image."""
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.common.utils import flatten_items, tree_map
from axlearn_b200.vision import rcnn
from axlearn_b200.vision.resnet import named_resnet_config


def test_roi_levels_and_multilevel_align():
    boxes = torch.tensor([[0, 0, 32, 32], [0, 0, 224, 224], [0, 0, 900, 900.0]])
    assert rcnn.roi_levels(boxes, min_level=2, max_level=5).tolist() == [2, 4, 5]
    feats = {2: torch.full((16, 16, 3), 2.0), 3: torch.full((8, 8, 3), 3.0)}
    out = rcnn.multilevel_roi_align(feats, torch.tensor([[0, 0, 20, 20], [0, 0, 120, 120.0]]), output_size=2)
    assert out.shape == (2, 2, 2, 3) and out[0].unique().tolist() == [2.0] and out[1].unique().tolist() == [3.0]


def test_proposals_are_decoded_clipped_and_suppressed():
    anchors = torch.tensor([[10, 10, 30, 30], [11, 11, 31, 31], [50, 50, 70, 70], [-20, -20, 5, 5.0]])
    scores = torch.tensor([0.9, 0.8, 0.7, 0.6])
    boxes, valid = rcnn.generate_proposals(scores=scores, deltas=torch.zeros(4, 4), anchors=anchors, image_shape=(64, 64),
                                           post_nms_top_k=4)
    assert valid.tolist() == [True, True, True, False]           # the near-duplicate is suppressed
    assert boxes[0].tolist() == [10, 10, 30, 30] and boxes[1].tolist() == [50, 50, 64, 64]
    assert boxes[2].tolist() == [0, 0, 5, 5]


def test_faster_rcnn_overfits_one_image_and_detects_its_box():
    torch.manual_seed(0)
    backbone = named_resnet_config("resnet18").set(hidden_dim=8, num_blocks_per_stage=(1, 1, 1, 1))
    cfg = rcnn.FasterRCNN.default_config().set(
        name="frcnn", backbone=backbone, num_classes=2, rpn_batch_size=64, roi_batch_size=32, pre_nms_top_k=200,
        post_nms_top_k=50, anchor_size=4.0)
    cfg.fpn.hidden_dim = 16
    cfg.rcnn_head.set(hidden_dim=64, roi_size=4)
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    image = torch.zeros(1, 128, 128, 3)
    image[0, 40:90, 30:100] = 1.0
    batch = dict(image=image, gt_boxes=torch.tensor([[[40, 30, 90, 100.0], [0, 0, 0, 0]]]), gt_classes=torch.tensor([[2, -1]]))
    params = tree_map(lambda p: p.clone().requires_grad_(p.is_floating_point()), params)
    leaves = [p for k, p in flatten_items(params) if p.requires_grad and "moving" not in k]
    opt = torch.optim.Adam(leaves, lr=2e-3)
    first = None
    for step in range(160):
        (loss, aux), _ = functional(model, prng.PRNGKey(step), params, [batch], is_training=True)
        first = first if first is not None else loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert set(aux) == {"rpn_score_loss", "rpn_box_loss", "frcnn_class_loss", "frcnn_box_loss"}
    assert loss.item() < 0.5 * first
    out, _ = functional(model, None, params, dict(input_batch=dict(image=image)), is_training=True, method="predict")
    assert int(out["num_detections"][0]) >= 1
    assert int(out["detection_classes"][0, 0]) == 2
    from axlearn_b200.vision.detection_utils import pairwise_iou
    assert pairwise_iou(out["detection_boxes"][0, :1], batch["gt_boxes"][0, :1])[0, 0] > 0.5
