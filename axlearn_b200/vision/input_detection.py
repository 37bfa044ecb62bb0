"""Detection input processing: RetinaNet-style resize / pad, box bookkeeping, fixed-size labels
(reference: axlearn/vision/input_detection.py:26-516, utils_detection.py box helpers).

Examples are dicts with ``image [H, W, 3]`` (uint8 or float), ``groundtruth_boxes [N, 4]``
(normalised ``ymin, xmin, ymax, xmax``), ``groundtruth_classes [N]``, ``groundtruth_is_crowd [N]``,
``groundtruth_area [N]``, ``source_id``, ``height``, ``width``.  Everything here is host-side numpy
(deterministic under a ``numpy.random.Generator``) and plugs into ``input_pipeline`` stages;
batches reach the GPU through the pinned-tensor path of ``PipelineInput``.
"""

from __future__ import annotations

import zlib
from typing import Callable, Optional, Sequence

import numpy as np

from axlearn_b200.common import input_pipeline
from axlearn_b200.common.config import config_class
from axlearn_b200.vision.input_image import resize_bilinear, whiten

Rng = Optional[np.random.Generator]


def random_horizontal_flip(image: np.ndarray, boxes: np.ndarray, rng: Rng = None) -> tuple[np.ndarray, np.ndarray]:
    """Flips image and (normalised) boxes left-right with probability one half."""
    rng = rng or np.random.default_rng()
    if rng.uniform() <= 0.5:
        return image, boxes
    flipped = boxes.copy()
    flipped[:, 1] = 1.0 - boxes[:, 3]
    flipped[:, 3] = 1.0 - boxes[:, 1]
    return image[:, ::-1].copy(), flipped


def compute_padded_size(desired_size: Sequence[int], stride: int) -> tuple[int, int]:
    """Smallest multiples of ``stride`` that hold ``desired_size``."""
    return tuple(int(-(-s // stride) * stride) for s in desired_size)


def resize_and_crop_image(image: np.ndarray, *, desired_size: Sequence[int], padded_size: Sequence[int],
                          aug_scale_min: float = 1.0, aug_scale_max: float = 1.0,
                          rng: Rng = None) -> tuple[np.ndarray, np.ndarray]:
    """Keeps the aspect ratio, scales the image to the largest size inside ``desired_size``
    (times a random factor in ``[aug_scale_min, aug_scale_max]`` when they differ from 1, followed
    by a random crop back to ``desired_size``), then zero-pads at the bottom / right to
    ``padded_size``.  Returns the image and ``image_info`` ``[[orig_h, orig_w], [desired_h,
    desired_w], [y_scale, x_scale], [y_offset, x_offset]]``."""
    image_size = np.asarray(image.shape[:2], dtype=np.float32)
    desired = np.asarray(desired_size, dtype=np.float32)
    jitter = aug_scale_min != 1.0 or aug_scale_max != 1.0
    if jitter:
        rng = rng or np.random.default_rng()
        scaled = np.round(rng.uniform(aug_scale_min, aug_scale_max) * desired)
    else:
        scaled = desired
    scale = min(scaled[0] / image_size[0], scaled[1] / image_size[1])
    scaled = np.round(image_size * scale)
    image_scale = scaled / image_size
    offset = np.zeros(2, dtype=np.int32)
    if jitter:
        max_offset = np.maximum(scaled - desired, 0)
        offset = (max_offset * rng.uniform(size=2)).astype(np.int32)
    out = resize_bilinear(image.astype(np.float32), (int(scaled[0]), int(scaled[1])))
    if jitter:
        out = out[offset[0]:offset[0] + int(desired[0]), offset[1]:offset[1] + int(desired[1])]
    padded = np.zeros((padded_size[0], padded_size[1], image.shape[2]), dtype=np.float32)
    padded[:out.shape[0], :out.shape[1]] = out
    info = np.stack([image_size, desired, image_scale.astype(np.float32), offset.astype(np.float32)])
    return padded, info


def denormalize_boxes(boxes: np.ndarray, image_shape: Sequence[int]) -> np.ndarray:
    h, w = float(image_shape[0]), float(image_shape[1])
    return boxes.astype(np.float32) * np.asarray([h, w, h, w], dtype=np.float32)


def normalize_boxes(boxes: np.ndarray, image_shape: Sequence[int]) -> np.ndarray:
    h, w = float(image_shape[0]), float(image_shape[1])
    return boxes.astype(np.float32) / np.asarray([h, w, h, w], dtype=np.float32)


def resize_and_crop_boxes(boxes: np.ndarray, image_scale: np.ndarray, output_size: np.ndarray,
                          offset: np.ndarray) -> np.ndarray:
    """Applies the image's scale and crop offset to pixel boxes and clips them to the output."""
    boxes = boxes * np.tile(image_scale, 2) - np.tile(offset, 2)
    limit = np.tile(np.asarray(output_size, dtype=np.float32), 2)
    return np.clip(boxes, 0.0, limit)


def get_non_empty_box_indices(boxes: np.ndarray) -> np.ndarray:
    return np.nonzero((boxes[:, 2] - boxes[:, 0] > 0) & (boxes[:, 3] - boxes[:, 1] > 0))[0]


def clip_or_pad_to_fixed_size(x: np.ndarray, size: int, constant_value=0) -> np.ndarray:
    """First ``size`` rows of ``x``, padded with ``constant_value`` rows when there are fewer."""
    x = np.asarray(x)[:size]
    pad = size - x.shape[0]
    if pad == 0:
        return x
    fill = np.full((pad,) + x.shape[1:], constant_value, dtype=x.dtype)
    return np.concatenate([x, fill], axis=0)


def process_source_id(source_id) -> np.int64:
    """Numeric ids are kept; other strings are hashed to a stable 31-bit number."""
    if isinstance(source_id, (bytes, np.bytes_)):
        source_id = source_id.decode()
    if isinstance(source_id, str):
        return np.int64(int(source_id)) if source_id.isdigit() else np.int64(zlib.crc32(source_id.encode()) & 0x7FFFFFFF)
    return np.int64(source_id)


def parse_train_example(data: dict, *, output_size: Sequence[int], output_stride: int, aug_scale_min: float,
                        aug_scale_max: float, aug_rand_hflip: bool = True, skip_crowd_during_training: bool = True,
                        max_num_instances: int = 100, rng: Rng = None) -> dict:
    classes = np.asarray(data["groundtruth_classes"])
    boxes = np.asarray(data["groundtruth_boxes"], dtype=np.float32).reshape(-1, 4)
    crowds = np.asarray(data.get("groundtruth_is_crowd", np.zeros(len(classes), dtype=bool))).astype(bool)
    if skip_crowd_during_training and crowds.size:
        keep = np.nonzero(~crowds)[0]
        classes, boxes = classes[keep], boxes[keep]
    image = whiten(np.asarray(data["image"]))
    shape = image.shape[:2]
    if aug_rand_hflip:
        image, boxes = random_horizontal_flip(image, boxes, rng)
    boxes = denormalize_boxes(boxes, shape)
    image, info = resize_and_crop_image(image, desired_size=output_size,
                                        padded_size=compute_padded_size(output_size, output_stride),
                                        aug_scale_min=aug_scale_min, aug_scale_max=aug_scale_max, rng=rng)
    boxes = resize_and_crop_boxes(boxes, info[2], info[1], info[3])
    keep = get_non_empty_box_indices(boxes)
    boxes, classes = boxes[keep], classes[keep]
    return {"image_data": {"image": image, "image_info": info},
            "labels": {"groundtruth_boxes": clip_or_pad_to_fixed_size(boxes.astype(np.float32), max_num_instances, -1),
                       "groundtruth_classes": clip_or_pad_to_fixed_size(classes.astype(np.int32), max_num_instances, -1)}}


def parse_eval_example(data: dict, *, output_size: Sequence[int], output_stride: int, max_num_instances: int = 100,
                       **unused) -> dict:
    del unused
    classes = np.asarray(data["groundtruth_classes"])
    boxes = np.asarray(data["groundtruth_boxes"], dtype=np.float32).reshape(-1, 4)
    image = whiten(np.asarray(data["image"]))
    shape = image.shape[:2]
    image, info = resize_and_crop_image(image, desired_size=output_size,
                                        padded_size=compute_padded_size(output_size, output_stride))
    n = len(classes)
    crowds = np.asarray(data.get("groundtruth_is_crowd", np.zeros(n, dtype=bool))).astype(np.int32)
    areas = np.asarray(data.get("groundtruth_area", np.zeros(n, dtype=np.float32)), dtype=np.float32)
    gt = {
        "source_id": process_source_id(data.get("source_id", 0)),
        "height": np.int32(data.get("height", shape[0])), "width": np.int32(data.get("width", shape[1])),
        "num_detections": np.int32(n), "image_info": info,
        # Evaluation compares in the ORIGINAL image's pixel coordinates.
        "boxes": clip_or_pad_to_fixed_size(denormalize_boxes(boxes, shape), max_num_instances, -1),
        "classes": clip_or_pad_to_fixed_size(classes.astype(np.int32), max_num_instances, -1),
        "areas": clip_or_pad_to_fixed_size(areas, max_num_instances, -1),
        "is_crowds": clip_or_pad_to_fixed_size(crowds, max_num_instances, 0),
    }
    return {"image_data": {"image": image, "image_info": info}, "labels": {"groundtruths": gt}}


def detection_processor(*, is_training: bool, image_size: Sequence[int], output_stride: int = 128,
                        max_num_instances: int = 100, aug_scale_min: float = 1.0, aug_scale_max: float = 1.0,
                        aug_rand_hflip: bool = True, seed: int = 0) -> Callable[[dict], dict]:
    """A per-example function for ``Stage.map``.  Training augmentation draws from a generator
    seeded by ``(seed, example counter)``, so a restored pipeline repeats the same crops."""
    counter = {"n": 0}

    def fn(example: dict) -> dict:
        if not is_training:
            return parse_eval_example(example, output_size=image_size, output_stride=output_stride,
                                      max_num_instances=max_num_instances)
        rng = np.random.default_rng((seed, example.get("_index", counter["n"])))
        counter["n"] += 1
        return parse_train_example(example, output_size=image_size, output_stride=output_stride,
                                   aug_scale_min=aug_scale_min, aug_scale_max=aug_scale_max,
                                   aug_rand_hflip=aug_rand_hflip, max_num_instances=max_num_instances, rng=rng)

    return fn


class DetectionInput(input_pipeline.PipelineInput):
    """``source`` yields raw detection examples; this input parses, augments and batches them
    (reference ``DetectionInput``, :447-474)."""

    @config_class
    class Config(input_pipeline.PipelineInput.Config):
        image_size: Sequence[int] = (640, 640)
        output_stride: int = 128
        max_num_instances: int = 100
        aug_scale_min: float = 1.0
        aug_scale_max: float = 1.0
        aug_rand_hflip: bool = True
        seed: int = 0

    def _make_source(self):
        cfg = self._config
        raw_source = super()._make_source()
        proc = detection_processor(
            is_training=cfg.is_training, image_size=cfg.image_size, output_stride=cfg.output_stride,
            max_num_instances=cfg.max_num_instances, aug_scale_min=cfg.aug_scale_min,
            aug_scale_max=cfg.aug_scale_max, aug_rand_hflip=cfg.aug_rand_hflip, seed=cfg.seed)
        return lambda index, count: raw_source(index, count).map(proc)


def fake_detection_source(*, num_examples: int = 8, image_size: Sequence[int] = (96, 128), max_boxes: int = 5,
                          num_classes: int = 10, seed: int = 0):
    """``source(shard_index, shard_count)`` of synthetic detection examples (the counterpart of
    the reference's ``fake_detection_dataset``, :476-516)."""

    def make(index: int, count: int):
        rng = np.random.default_rng(seed)
        rows = []
        for i in range(num_examples):
            n = int(rng.integers(1, max_boxes + 1))
            y0, x0 = rng.uniform(0, 0.6, n), rng.uniform(0, 0.6, n)
            hh, ww = rng.uniform(0.1, 0.4, n), rng.uniform(0.1, 0.4, n)
            boxes = np.stack([y0, x0, np.minimum(y0 + hh, 1.0), np.minimum(x0 + ww, 1.0)], axis=1).astype(np.float32)
            rows.append({
                "image": rng.integers(0, 256, (image_size[0], image_size[1], 3), dtype=np.uint8),
                "groundtruth_boxes": boxes,
                "groundtruth_classes": rng.integers(1, num_classes, n).astype(np.int64),
                "groundtruth_is_crowd": rng.uniform(size=n) < 0.1,
                "groundtruth_area": ((boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1])
                                     * image_size[0] * image_size[1]).astype(np.float32),
                "source_id": str(1000 + i), "height": image_size[0], "width": image_size[1], "_index": i,
            })
        return input_pipeline.read(input_pipeline.ListSource(rows), shard_index=index, shard_count=count,
                                   num_epochs=None)

    return make
