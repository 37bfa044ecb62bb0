"""Box coder, anchors and anchor labelling, box utilities."""

import itertools

import numpy as np
import pytest
import torch

from axlearn_b200.vision import anchor, box_coder, matchers
from axlearn_b200.vision import utils_detection as ud


def test_box_coder_round_trip_and_clipping():
    gen = torch.Generator().manual_seed(0)
    yx = torch.rand(2, 50, 2, generator=gen) * 100
    anchors = torch.cat([yx, yx + torch.rand(2, 50, 2, generator=gen) * 50 + 5], -1)
    yx2 = torch.rand(2, 50, 2, generator=gen) * 100
    boxes = torch.cat([yx2, yx2 + torch.rand(2, 50, 2, generator=gen) * 50 + 5], -1)
    coder = box_coder.BoxCoder.default_config().set(weights=(10.0, 10.0, 5.0, 5.0)).instantiate()
    enc = coder.encode(boxes=boxes, anchors=anchors)
    torch.testing.assert_close(coder.decode(encoded_boxes=enc, anchors=anchors), boxes, atol=1e-3, rtol=1e-4)
    # A box equal to its anchor encodes to zeros.
    torch.testing.assert_close(coder.encode(boxes=anchors, anchors=anchors), torch.zeros_like(anchors), atol=1e-6, rtol=0)
    # Hand check: box twice the anchor's size, shifted by half the anchor's height.
    a = torch.tensor([[0.0, 0.0, 10.0, 10.0]])
    b = torch.tensor([[-5.0, -5.0, 15.0, 15.0]]) + torch.tensor([[5.0, 0.0, 5.0, 0.0]])
    plain = box_coder.BoxCoder.default_config().instantiate()
    torch.testing.assert_close(plain.encode(boxes=b, anchors=a), torch.tensor([[0.5, 0.0, np.log(2.0), np.log(2.0)]]).float(),
                               atol=1e-6, rtol=1e-6)
    huge = torch.tensor([[0.0, 0.0, 100.0, 100.0]])
    h = plain.decode(encoded_boxes=huge, anchors=a)
    assert torch.isfinite(h).all() and abs((h[0, 2] - h[0, 0]).item() - 10 * box_coder.BBOX_XFORM_CLIP_EXP) < 1e-2
    unclipped = box_coder.BoxCoder.default_config().set(clip_boxes=box_coder.BoxClipMethod.NONE).instantiate()
    assert torch.isinf(unclipped.decode(encoded_boxes=huge, anchors=a)).any()
    both = box_coder.BoxCoder.default_config().set(clip_boxes=box_coder.BoxClipMethod.MinMaxYXHW).instantiate()
    d = both.decode(encoded_boxes=torch.tensor([[1e6, -1e6, -100.0, 0.0]]), anchors=a)
    assert abs((d[0, 0] + d[0, 2]).item() / 2 - (5 + 10 * box_coder.BBOX_XFORM_CLIP_EXP)) < 1e-2


def test_anchor_generator_layout():
    gen = anchor.AnchorGenerator(min_level=3, max_level=4, num_scales=2, aspect_ratios=(1.0, 2.0), anchor_size=4.0)
    anchors = gen((32, 64))
    assert list(anchors) == ["3", "4"] and anchors["3"].shape == (4 * 8 * 4, 4) and anchors["4"].shape == (2 * 4 * 4, 4)
    # First cell of level 3: centre (4, 4); (scale 0, aspect 1), (scale 0, aspect 2), (scale 1, aspect 1), ...
    a = anchors["3"][:4]
    torch.testing.assert_close(a[0], torch.tensor([4 - 16.0, 4 - 16.0, 4 + 16.0, 4 + 16.0]))
    w, h = a[1, 3] - a[1, 1], a[1, 2] - a[1, 0]
    assert abs((w / h).item() - 2.0) < 1e-5 and abs((w * h).item() - 32.0 ** 2) < 1e-2     # aspect = width / height
    assert abs(((a[2, 2] - a[2, 0]) / 32.0).item() - 2 ** 0.5) < 1e-5
    # Second cell is one stride to the right.
    torch.testing.assert_close(anchors["3"][4], a[0] + torch.tensor([0.0, 8.0, 0.0, 8.0]))


def test_anchor_labeler():
    per_level = {"3": torch.tensor([[0.0, 0.0, 10.0, 10.0], [0.0, 10.0, 10.0, 20.0]]),
                 "4": torch.tensor([[0.0, 0.0, 20.0, 20.0], [50.0, 50.0, 60.0, 60.0]])}
    gt_boxes = torch.tensor([[[0.0, 0.0, 10.0, 10.0], [0.0, 10.0, 10.0, 17.0], [-1.0, -1.0, -1.0, -1.0]]])
    gt_classes = torch.tensor([[3, 7, -1]])
    labeler = anchor.AnchorLabeler(matchers.ArgmaxMatcher.default_config().set(
        thresholds=[0.3, 0.6], labels=[matchers.BACKGROUND, matchers.IGNORE, matchers.FOREGROUND], force_match_columns=False))
    out = labeler(per_level_anchor_boxes=per_level, groundtruth_boxes=gt_boxes, groundtruth_classes=gt_classes)
    # Anchor 0 = gt 0 exactly; anchor 1 overlaps gt 1 with IoU 0.7; anchor 2 has IoU 0.25 (background);
    # anchor 3 overlaps nothing.
    assert out.groundtruth_classes.tolist() == [[3, 7, -1, -1]]
    assert out.box_paddings.tolist() == [[False, False, True, True]]
    assert out.class_paddings.tolist() == [[False, False, False, False]]
    torch.testing.assert_close(out.groundtruth_boxes[0, 1], gt_boxes[0, 1])
    assert not out.groundtruth_boxes[0, 2:].any() and out.anchor_boxes.shape == (4, 4)
    # Multi-label classes keep their trailing dimension.
    multi = torch.tensor([[[1, 0], [0, 1], [0, 0]]])
    out2 = labeler(per_level_anchor_boxes=per_level, groundtruth_boxes=gt_boxes, groundtruth_classes=multi)
    assert out2.groundtruth_classes.tolist() == [[[1, 0], [0, 1], [-1, -1], [-1, -1]]]


def test_box_utilities():
    boxes = torch.tensor([[[10.0, 20.0, 30.0, 60.0], [-5.0, 0.0, 120.0, 300.0]]])
    norm = ud.normalize_boxes(boxes=boxes, image_shape=[100, 200])
    torch.testing.assert_close(norm[0, 0], torch.tensor([0.1, 0.1, 0.3, 0.3]))
    torch.testing.assert_close(ud.denormalize_boxes(boxes=norm, image_shape=torch.tensor([[[100, 200]]])), boxes)
    assert ud.clip_boxes(boxes, [100, 200])[0, 1].tolist() == [0.0, 0.0, 100.0, 200.0]
    with pytest.raises(ValueError):
        ud.clip_boxes(torch.zeros(2, 3), [1, 1])
    assert ud.sorted_top_k(torch.tensor([[1.0, 5.0, 3.0, 5.0]]), k=3).tolist() == [[3, 1, 2]]
    out = ud.resize_and_crop_boxes(boxes[0], torch.tensor([0.5, 2.0]), [50, 100], torch.tensor([5.0, 10.0]))
    assert out[0].tolist() == [0.0, 30.0, 10.0, 100.0]
    assert ud.get_non_empty_box_indices(torch.tensor([[0.0, 0, 1, 1], [0, 0, 0, 1], [1, 1, 2, 3]])).tolist() == [0, 2]
    assert ud.compute_padded_size((100, 200), 32) == [128, 224]
    assert ud.process_source_id("42") == 42 and ud.process_source_id(b"") == -1 and ud.process_source_id(7) == 7
    flat = ud.multi_level_flatten({3: torch.zeros(2, 4, 4, 8), 4: torch.ones(2, 2, 2, 8)}, last_dim=4)
    assert flat.shape == (2, 4 * 4 * 2 + 2 * 2 * 2, 4)
    assert ud.multi_level_flatten({3: torch.zeros(2, 4, 4), 4: torch.ones(2, 2, 2)}).shape == (2, 20)
    assert ud.clip_or_pad_to_fixed_size(torch.arange(3), 5, -1).tolist() == [0, 1, 2, -1, -1]
    assert ud.clip_or_pad_to_fixed_size(torch.arange(6).reshape(3, 2), 2).tolist() == [[0, 1], [2, 3]]
    gts = ud.pad_groundtruths_to_fixed_size({"boxes": torch.ones(1, 4), "is_crowds": torch.ones(1), "areas": torch.ones(1),
                                             "classes": torch.ones(1), "source_id": 3}, 2)
    assert gts["boxes"].tolist() == [[1.0] * 4, [-1.0] * 4] and gts["is_crowds"].tolist() == [1.0, 0.0] and gts["source_id"] == 3
    fb, fs = ud.filter_boxes_by_scores(boxes[0], torch.tensor([0.9, 0.1]), 0.5)
    assert fb[1].tolist() == [0.0] * 4 and fs.tolist() == [pytest.approx(0.9), -1.0]
    assert ud.yxyx_to_xywh(np.array([[1.0, 2.0, 4.0, 8.0]])).tolist() == [[2.0, 1.0, 6.0, 3.0]]


def test_transform_boxes_all_pairs():
    b = torch.tensor([[1.0, 2.0, 4.0, 8.0]])
    F = ud.BoxFormat
    assert ud.transform_boxes(b, F.YminXminYmaxXmax, F.XminYminXmaxYmax).tolist() == [[2.0, 1.0, 8.0, 4.0]]
    assert ud.transform_boxes(b, F.YminXminYmaxXmax, F.XminYminWH).tolist() == [[2.0, 1.0, 6.0, 3.0]]
    assert ud.transform_boxes(b, F.YminXminYmaxXmax, F.CxCyWH).tolist() == [[5.0, 2.5, 6.0, 3.0]]
    assert ud.transform_boxes(torch.tensor([[2.0, 1.0, 6.0, 3.0]]), F.XminYminWH, F.YminXminHW).tolist() == [[1.0, 2.0, 3.0, 6.0]]
    for src, dst in itertools.product(F, F):
        there = ud.transform_boxes(b, F.YminXminYmaxXmax, src)
        torch.testing.assert_close(ud.transform_boxes(ud.transform_boxes(there, src, dst), dst, F.YminXminYmaxXmax), b)

    @ud.reshape_box_decorator
    def heights(bx):
        assert bx.ndim == 2
        return bx[:, 2] - bx[:, 0]

    assert heights(torch.zeros(2, 3, 4)).shape == (2, 3)
