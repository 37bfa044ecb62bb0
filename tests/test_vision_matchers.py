"""Matchers, similarity ops and samplers (vectors: axlearn/vision/matchers_test.py:15-185)."""

import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.vision import matchers, samplers, similarity_ops


def _t(x):
    return torch.tensor(x, dtype=torch.float32)


def test_similarity_ops():
    a = _t([[[0, 0, 2, 2], [1, 1, 3, 3], [-1, -1, -1, -1]]])
    b = _t([[[0, 0, 2, 2], [2, 2, 4, 4]]])
    iou = similarity_ops.pairwise_iou(boxes_a=a, boxes_b=b, paddings_a=a.amax(-1) < 0)
    torch.testing.assert_close(iou, _t([[[1.0, 0.0], [1 / 7, 1 / 7], [-1.0, -1.0]]]))
    ioa = similarity_ops.pairwise_ioa(boxes_a=a[:, :2], boxes_b=b)
    torch.testing.assert_close(ioa, _t([[[1.0, 0.0], [0.25, 0.25]]]))
    e = similarity_ops.elementwise_iou(boxes_a=a[:, :2], boxes_b=b, paddings_b=torch.tensor([[False, True]]), fill_value=-3.0)
    torch.testing.assert_close(e, _t([[1.0, -3.0]]))
    # Degenerate boxes: no division by an empty union.
    z = _t([[[0, 0, 0, 0]]])
    assert similarity_ops.pairwise_iou(boxes_a=z, boxes_b=z).item() == 0.0
    assert similarity_ops.areas(a).tolist() == [[4.0, 4.0, 0.0]]


def test_argmax_only_high_quality_matches():
    anchors = {"all": _t([[0, 0, 1, 0.3], [0, 0.5, 1, 1]])}
    gt = _t([[[0, 0.26, 1, 1], [0, 0, 0, 0], [0, 0.5, 1, 1], [0, 0, 0, 0]],
             [[0, 0, 0, 0], [0, 0, 0.02, 0.02], [0, 0, 0, 0], [0, 0.3, 1, 0.8]]])
    m = matchers.ArgmaxMatcher.default_config().set(thresholds=[0.01, 0.2, 0.5], labels=[-2, -1, 0, 1],
                                                    force_match_columns=False).instantiate()
    r = m.match(per_level_anchor_boxes=anchors, groundtruth_boxes=gt)
    assert r.matches.tolist() == [[0, 2], [1, 3]] and r.labels.tolist() == [[-1, 1], [-2, 0]]
    assert r.anchor_boxes.shape == (1, 2, 4)


def test_argmax_forced_matches():
    anchors = {"all": _t([[0, 0.5, 0.5, 0.85], [0, 0, 0.4, 0.5], [0.5, 0.5, 0.55, 1], [0, 0.5, 0.1, 1],
                          [0.5, 0, 0.75, 0.5], [0, 0.5, 0.2, 1], [0, 0.5, 0.1, 1], [0, 0, 0.05, 0.5]])}
    gt = _t([[[0, 0, 0.5, 0.5], [0, 0.5, 0.5, 1], [0.5, 0, 1, 0.5], [0.5, 0.5, 1, 1]]])
    m = matchers.ArgmaxMatcher.default_config().set(thresholds=[0.0, 0.3, 0.6], labels=[-2, -1, 0, 1]).instantiate()
    r = m.match(per_level_anchor_boxes=anchors, groundtruth_boxes=gt)
    assert r.matches.tolist() == [[1, 0, 3, 1, 2, 1, 1, 0]]
    assert r.labels.tolist() == [[1, 1, 1, -1, 1, 0, -1, -1]]
    with pytest.raises(ValueError):
        matchers.ArgmaxMatcher.default_config().set(thresholds=[0.5], labels=[-1, 1, 2, 3]).instantiate()
    with pytest.raises(ValueError):
        matchers.ArgmaxMatcher.default_config().set(thresholds=[0.6, 0.5]).instantiate()


@pytest.mark.parametrize("mode", [matchers.DistanceType.L2, matchers.DistanceType.IOU])
def test_atss_matches(mode):
    anchors = {"2": _t([[0, 0, 0.5, 0.5], [0, 0.5, 0.5, 1], [0.5, 0, 1, 0.5], [0.5, 0.5, 1, 1]]),
               "3": _t([[0, 0, 1, 0.5], [0, 0, 0.5, 1], [0, 0.5, 1, 1], [0.5, 0, 1, 1]])}
    gt = _t([[[0, 0, 0.5, 0.5], [0, 0, 0.5, 1]]])
    m = matchers.ATSSMatcher.default_config().set(top_k=3, distance_type=mode, labels=[-1, 0, 1]).instantiate()
    r = m.match(anchors, gt)
    assert r.matches.tolist() == [[0, 1, 0, 0, 0, 1, 1, 0]]
    assert r.labels.tolist() == [[1, -1, -1, -1, -1, 1, -1, -1]]


def test_atss_labels_on_a_grid():
    lvl2 = [[0.0, 0.0, 256.0, 256.0], [256.0, 0.0, 512.0, 256.0], [0.0, 256.0, 256.0, 512.0], [256.0, 256.0, 512.0, 512.0]]
    lvl3 = [[float(y), float(x), float(y + 128), float(x + 128)] for (y, x) in
            [(0, 0), (128, 0), (0, 128), (128, 128), (0, 256), (128, 256), (0, 384), (128, 384), (256, 0), (384, 0),
             (256, 128), (384, 128), (256, 256), (384, 256), (256, 384), (384, 384)]]
    gt = _t([[[26.117289, 17.156782, 406.18396, 228.53214], [349.10214, 123.73946, 386.32037, 151.13103],
              [381.43216, 133.47852, 406.7317, 157.99454], [138.24228, 73.86143, 159.00032, 90.12147],
              [125.70181, 70.05465, 143.48924, 84.57509]]])
    m = matchers.ATSSMatcher.default_config().set(top_k=3, labels=[-1, 0, 1]).instantiate()
    r = m.match({"2": _t(lvl2), "3": _t(lvl3)}, gt)
    assert r.labels.tolist() == [[1, -1, -1, -1, -1, 1, -1, -1, -1, -1, -1, -1, -1, -1, 1, -1, -1, -1, -1, -1]]


def test_sample_and_label_sampler():
    key = prng.PRNGKey(0)
    cand = torch.tensor([[True, False, True, True, False, True], [False, False, True, False, False, False]])
    picked = samplers.sample(is_candidate=cand, size=torch.tensor([2, 3]), prng_key=key)
    assert picked.sum(-1).tolist() == [2, 1] and not (picked & ~cand).any()
    labels = torch.tensor([[1, 1, 1, 1, -1, -1, -1, -2, -1, 5], [1, -1, -1, -2, -2, -1, 0, 0, 0, 0]])
    paddings = torch.tensor([[False] * 10, [False] * 6 + [True] * 4])
    sampler = samplers.LabelSampler(size=6, foreground_fraction=0.5, background_label=-1, ignore_label=-2)
    out = sampler(labels=labels, paddings=paddings, prng_key=key)
    assert out.indices.shape == (2, 6) and out.paddings.shape == (2, 6)
    # Row 0: three foreground (of five) and three background (of four), none ignored.
    chosen = labels[0][out.indices[0][~out.paddings[0]]]
    assert (chosen > 0).sum() == 3 and (chosen == -1).sum() == 3
    # Row 1: one foreground, all three background; the rest of the sample is filler.
    chosen = labels[1][out.indices[1][~out.paddings[1]]]
    assert sorted(chosen.tolist()) == [-1, -1, -1, 1] and out.paddings[1].sum() == 2
    # Deterministic for a key, different across keys.
    again = sampler(labels=labels, paddings=paddings, prng_key=key)
    assert torch.equal(again.indices, out.indices)
