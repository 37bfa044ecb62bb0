"""BiFPN / EfficientDet shapes and a training step; COCO metrics on hand-checkable cases."""
import numpy as np
import pytest
import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.vision import efficientdet
from axlearn_b200.vision.coco_evaluator import COCOEvaluator


def test_weighted_fusion_normalises_its_weights():
    for method in ("attention", "fastattention", "sum"):
        layer = efficientdet.WeightedFeatureFusion.default_config().set(name="f", num_inputs=2, method=method).instantiate(parent=None)
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
        a, b = torch.ones(1, 2, 2, 3), 3 * torch.ones(1, 2, 2, 3)
        y, _ = functional(layer, None, params, [[a, b]], is_training=False)
        want = 4.0 if method == "sum" else 2.0
        torch.testing.assert_close(y, torch.full_like(a, want), rtol=1e-3, atol=1e-3)


def test_efficientdet_test_variant_trains_a_step():
    cfg = efficientdet.efficientdet_config("test", num_classes=3).set(name="det")
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    size = efficientdet.image_size("test")
    batch = dict(image=torch.randn(2, size, size, 3),
                 groundtruth_boxes=torch.tensor([[[4, 4, 40, 40.0]], [[10, 20, 50, 60.0]]]),
                 groundtruth_classes=torch.tensor([[1], [2]]))
    (loss, out), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True)
    anchors = sum((size // 2 ** l) ** 2 * 9 for l in range(3, 8))
    assert out["class_outputs"].shape == (2, anchors, 3) and out["box_outputs"].shape == (2, anchors, 4)
    assert torch.isfinite(loss)
    d0 = efficientdet.efficientdet_config("d0")
    assert d0.fpn.hidden_dim == 64 and d0.fpn.num_layers == 3 and d0.head.num_layers == 3
    assert efficientdet.efficientdet_config("d4").fpn.hidden_dim == 224 and efficientdet.image_size("d7") == 1536


def test_coco_metrics_perfect_and_half():
    ev = COCOEvaluator()
    gt = np.array([[10, 10, 60, 60], [100, 100, 180, 220.0]])
    ev.add_groundtruth("a", gt, [1, 2])
    ev.add_detections("a", gt, [0.9, 0.8], [1, 2])
    m = ev.evaluate()
    assert m["AP"] == pytest.approx(1.0) and m["AP50"] == pytest.approx(1.0) and m["ARmax100"] == pytest.approx(1.0)
    assert m["APm"] == pytest.approx(1.0) and m["APl"] == pytest.approx(1.0) and m["APs"] == -1.0

    ev.reset()
    ev.add_groundtruth("a", gt[:1], [1])
    ev.add_groundtruth("b", gt[:1], [1])
    ev.add_detections("a", gt[:1], [0.9], [1])                      # one of two found, no false positives
    m = ev.evaluate()
    assert m["AP50"] == pytest.approx(51 / 101, abs=1e-6) and m["ARmax100"] == pytest.approx(0.5)

    ev.reset()
    ev.add_groundtruth("a", gt[:1], [1])
    shifted = np.array([[10, 10, 60, 50.0]])                        # IoU 0.8: counts up to threshold 0.80
    ev.add_detections("a", shifted, [0.9], [1])
    m = ev.evaluate()
    assert m["AP50"] == pytest.approx(1.0) and m["AP75"] == pytest.approx(1.0)
    assert m["AP"] == pytest.approx(0.7, abs=1e-6)

    ev.reset()                                                      # a higher-scored false positive halves precision
    ev.add_groundtruth("a", gt[:1], [1])
    ev.add_detections("a", np.array([[200, 200, 250, 250.0], [10, 10, 60, 60]]), [0.95, 0.9], [1, 1])
    assert ev.evaluate()["AP50"] == pytest.approx(0.5)

    ev.reset()                                                      # crowd regions absorb detections silently
    ev.add_groundtruth("a", gt, [1, 1], is_crowd=[False, True])
    ev.add_detections("a", gt, [0.9, 0.8], [1, 1])
    assert ev.evaluate()["AP50"] == pytest.approx(1.0)
