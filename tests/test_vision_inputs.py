"""Detection / image-classification input processing and detection drawing."""

import numpy as np
import pytest
import torch

from axlearn_b200.vision import input_detection as det
from axlearn_b200.vision import input_image as img
from axlearn_b200.vision import utils_visualization as vis


def test_whiten_roundtrip_and_resize_matches_torch():
    rng = np.random.default_rng(0)
    image = rng.integers(0, 256, (17, 23, 3), dtype=np.uint8)
    w = img.whiten(image)
    assert w.dtype == np.float32 and abs(float(w.mean())) < 1.5
    np.testing.assert_array_equal(img.de_whiten(w), image)
    got = img.resize_bilinear(image, (40, 31))
    ref = torch.nn.functional.interpolate(torch.from_numpy(image).permute(2, 0, 1)[None].float(), size=(40, 31),
                                          mode="bilinear", align_corners=False)[0].permute(1, 2, 0).numpy()
    np.testing.assert_allclose(got, ref, atol=1e-3)
    down = img.resize_bilinear(image, (9, 11))
    ref = torch.nn.functional.interpolate(torch.from_numpy(image).permute(2, 0, 1)[None].float(), size=(9, 11),
                                          mode="bilinear", align_corners=False)[0].permute(1, 2, 0).numpy()
    np.testing.assert_allclose(down, ref, atol=1e-3)


def test_crops():
    image = np.arange(20 * 30 * 3, dtype=np.float32).reshape(20, 30, 3)
    c = img.central_crop(image, (10, 10))
    np.testing.assert_array_equal(c, image[5:15, 10:20])
    c2 = img.central_crop_v2(image, 0.5)
    assert c2.shape == (10, 10, 3)
    rng = np.random.default_rng(1)
    for _ in range(20):
        r = img.random_crop(image, rng=rng)
        assert 0 < r.shape[0] <= 20 and 0 < r.shape[1] <= 30
        ratio = r.shape[1] / r.shape[0]
        assert r.shape[:2] == (20, 30) or 0.6 < ratio < 1.7
    tr = img.crop_augment_whiten(image, is_training=True, image_size=(8, 8), rng=np.random.default_rng(2))
    ev = img.crop_augment_whiten(image, is_training=False, image_size=(8, 8))
    ev2 = img.crop_augment_whiten(image, is_training=False, image_size=(8, 8), eval_resize=(10, 15))
    assert tr.shape == ev.shape == ev2.shape == (8, 8, 3)


def test_imagenet_input_batches_and_is_deterministic():
    def make(is_training):
        cfg = img.ImagenetInput.default_config().set(
            name="in", source=img.fake_image_source(num_examples=6), global_batch_size=4, is_training=is_training,
            image_size=(16, 16), num_classes=10, prefetch=0, pad_for_eval_num_batches=None)
        return cfg.instantiate(parent=None)

    a = next(iter(make(True).dataset()))
    b = next(iter(make(True).dataset()))
    assert a["image"].shape == (4, 3, 16, 16) and a["image"].dtype == torch.float32 and a["label"].shape == (4,)
    assert torch.equal(a["image"], b["image"])                   # same seed, same crops
    e = next(iter(make(False).dataset()))
    assert e["image"].shape[1:] == (3, 16, 16)
    assert not img.is_valid_image({"image": np.zeros((0, 4, 3))})


def test_flip_and_resize_keep_boxes_on_their_objects():
    image = np.zeros((50, 100, 3), dtype=np.float32)
    image[10:20, 60:90] = 1.0                                    # the object
    boxes = np.asarray([[0.2, 0.6, 0.4, 0.9]], dtype=np.float32)
    flipped = None
    for seed in range(20):                                       # find a draw that flips
        im2, b2 = det.random_horizontal_flip(image, boxes, np.random.default_rng(seed))
        if not np.array_equal(b2, boxes):
            flipped = (im2, b2)
            break
    assert flipped is not None
    im2, b2 = flipped
    np.testing.assert_allclose(b2, [[0.2, 0.1, 0.4, 0.4]], atol=1e-6)
    assert im2[10:20, 10:40].min() == 1.0 and im2[:, 45:].max() == 0.0
    out, info = det.resize_and_crop_image(image, desired_size=(64, 64), padded_size=det.compute_padded_size((64, 64), 128))
    assert out.shape == (128, 128, 3)
    np.testing.assert_allclose(info, [[50, 100], [64, 64], [0.64, 0.64], [0, 0]], atol=1e-6)
    assert out[40:, :].max() == 0.0                              # 50 * 0.64 = 32 rows of image, then padding
    px = det.resize_and_crop_boxes(det.denormalize_boxes(boxes, (50, 100)), info[2], info[1], info[3])
    np.testing.assert_allclose(px, [[6.4, 38.4, 12.8, 57.6]], atol=1e-4)
    y0, x0, y1, x1 = np.round(px[0]).astype(int)
    assert out[y0 + 1:y1 - 1, x0 + 1:x1 - 1].min() > 0.9         # the box still covers the object
    jit, info = det.resize_and_crop_image(image, desired_size=(64, 64), padded_size=(128, 128), aug_scale_min=1.5,
                                          aug_scale_max=2.0, rng=np.random.default_rng(0))
    assert jit.shape == (128, 128, 3) and 0.9 < info[2][0] and jit[64:, :].max() == 0.0 and jit[:, 64:].max() == 0.0


def test_train_and_eval_parsing_and_batches():
    src = det.fake_detection_source(num_examples=6, image_size=(48, 64), max_boxes=4)
    raw = next(src(0, 1))
    tr = det.parse_train_example(raw, output_size=(64, 64), output_stride=32, aug_scale_min=0.8, aug_scale_max=1.2,
                                 max_num_instances=7, rng=np.random.default_rng(0))
    assert tr["image_data"]["image"].shape == (64, 64, 3)
    gb, gc = tr["labels"]["groundtruth_boxes"], tr["labels"]["groundtruth_classes"]
    assert gb.shape == (7, 4) and gc.shape == (7,)
    valid = gc >= 0
    assert (gb[~valid] == -1).all() and (gb[valid][:, 2] > gb[valid][:, 0]).all() and gb[valid].max() <= 64
    ev = det.parse_eval_example(raw, output_size=(64, 64), output_stride=32, max_num_instances=7)
    gt = ev["labels"]["groundtruths"]
    n = int(gt["num_detections"])
    assert n == len(raw["groundtruth_classes"]) and gt["source_id"] == 1000 and gt["boxes"].shape == (7, 4)
    np.testing.assert_allclose(gt["boxes"][:n], det.denormalize_boxes(raw["groundtruth_boxes"], (48, 64)), atol=1e-4)
    cfg = det.DetectionInput.default_config().set(
        name="det", source=src, global_batch_size=2, image_size=(64, 64), output_stride=32, max_num_instances=5,
        aug_scale_min=0.9, aug_scale_max=1.1, prefetch=0)
    batch = next(iter(cfg.instantiate(parent=None).dataset()))
    assert batch["image_data"]["image"].shape == (2, 64, 64, 3)
    assert batch["labels"]["groundtruth_boxes"].shape == (2, 5, 4)
    again = next(iter(cfg.instantiate(parent=None).dataset()))
    assert torch.equal(batch["image_data"]["image"], again["image_data"]["image"])
    assert det.process_source_id("abc") == det.process_source_id(b"abc") and det.process_source_id("42") == 42
    np.testing.assert_array_equal(det.clip_or_pad_to_fixed_size(np.arange(3), 5, -1), [0, 1, 2, -1, -1])
    np.testing.assert_array_equal(det.clip_or_pad_to_fixed_size(np.arange(9), 5, -1), [0, 1, 2, 3, 4])


def test_visualize_detections(tmp_path):
    images = np.zeros((1, 20, 30, 3), dtype=np.uint8)
    boxes = np.asarray([[[2, 3, 10, 12], [5, 5, 8, 8], [0, 0, 19, 29]]], dtype=np.float32)
    scores = np.asarray([[0.9, 0.2, 0.8]])
    classes = np.asarray([[1, 2, -1]])
    out = vis.visualize_detections(images, boxes=boxes, scores=scores, classes=classes, thickness=1)
    assert (out[0, 2, 3:13] != 0).any(axis=-1).all() and (out[0, 2:11, 3] != 0).any(axis=-1).all()
    assert (out[0, 10, 3:13] != 0).any(axis=-1).all() and not out[0, 5, 5].any()      # low score: not drawn
    assert not out[0, 19, 20].any() and not images.any()                               # padded class; input untouched
    vis.write_ppm(str(tmp_path / "d.ppm"), out[0])
    raw = (tmp_path / "d.ppm").read_bytes()
    assert raw.startswith(b"P6\n30 20\n255\n") and len(raw) == 13 + 20 * 30 * 3
    img2 = vis.draw_box_on_image(np.zeros((10, 10, 3), np.uint8), [0.1, 0.1, 0.9, 0.9], normalized=True, thickness=1)
    assert img2[1, 1:10].any() and not img2[5, 5].any()
