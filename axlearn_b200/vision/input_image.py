"""Image-classification input processing (reference: axlearn/vision/input_image.py:51-438):
whitening, crops, the train / eval recipes of the ImageNet trainers, synthetic data.  Host-side
numpy on ``[H, W, C]`` images; the tensor augmentations (RandAugment, erasing, mixup) live in
``vision/augment.py`` and run on ``[C, H, W]`` tensors.
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence

import numpy as np

from axlearn_b200.common import input_pipeline
from axlearn_b200.common.config import config_class

Rng = Optional[np.random.Generator]

# Per-channel statistics of ImageNet in 0..255 units (the reference's whitening constants).
MEAN_RGB = (0.485 * 255, 0.456 * 255, 0.406 * 255)
STDDEV_RGB = (0.229 * 255, 0.224 * 255, 0.225 * 255)


def whiten(image: np.ndarray, mean_rgb: Sequence[float] = MEAN_RGB, stddev_rgb: Sequence[float] = STDDEV_RGB) -> np.ndarray:
    """``(image - mean) / stddev`` per channel, in float32."""
    return (image.astype(np.float32) - np.asarray(mean_rgb, np.float32)) / np.asarray(stddev_rgb, np.float32)


def de_whiten(image: np.ndarray, mean_rgb: Sequence[float] = MEAN_RGB, stddev_rgb: Sequence[float] = STDDEV_RGB) -> np.ndarray:
    """Inverse of ``whiten``, rounded and clipped back to uint8 (for visualisation)."""
    out = image.astype(np.float32) * np.asarray(stddev_rgb, np.float32) + np.asarray(mean_rgb, np.float32)
    return np.clip(np.round(out), 0, 255).astype(np.uint8)


def resize_bilinear(image: np.ndarray, size: Sequence[int]) -> np.ndarray:
    """Bilinear resize with half-pixel centres (no antialiasing), ``[H, W, C] -> [h, w, C]``."""
    h, w = image.shape[:2]
    oh, ow = int(size[0]), int(size[1])
    if (oh, ow) == (h, w):
        return image.astype(np.float32)
    ys = np.clip((np.arange(oh, dtype=np.float32) + 0.5) * (h / oh) - 0.5, 0, h - 1)
    xs = np.clip((np.arange(ow, dtype=np.float32) + 0.5) * (w / ow) - 0.5, 0, w - 1)
    y0, x0 = np.floor(ys).astype(np.int64), np.floor(xs).astype(np.int64)
    y1, x1 = np.minimum(y0 + 1, h - 1), np.minimum(x0 + 1, w - 1)
    wy, wx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
    img = image.astype(np.float32)
    top = img[y0][:, x0] * (1 - wx) + img[y0][:, x1] * wx
    bot = img[y1][:, x0] * (1 - wx) + img[y1][:, x1] * wx
    return top * (1 - wy) + bot * wy


def random_crop(image: np.ndarray, *, area_range=(0.08, 1.0), aspect_ratio_range=(3 / 4, 4 / 3),
                max_attempts: int = 10, rng: Rng = None) -> np.ndarray:
    """Inception-style crop: a window covering a random share of the area with a random aspect
    ratio; falls back to the whole image when no attempt fits."""
    rng = rng or np.random.default_rng()
    h, w = image.shape[:2]
    for _ in range(max_attempts):
        area = rng.uniform(*area_range) * h * w
        log_r = rng.uniform(np.log(aspect_ratio_range[0]), np.log(aspect_ratio_range[1]))
        ratio = float(np.exp(log_r))
        cw, ch = int(round(np.sqrt(area * ratio))), int(round(np.sqrt(area / ratio)))
        if 0 < cw <= w and 0 < ch <= h:
            y, x = int(rng.integers(0, h - ch + 1)), int(rng.integers(0, w - cw + 1))
            return image[y:y + ch, x:x + cw]
    return image


def central_crop(image: np.ndarray, image_size: Sequence[int]) -> np.ndarray:
    """Centre window of exactly ``image_size`` (the image must be at least that large)."""
    h, w = image.shape[:2]
    y, x = (h - image_size[0]) // 2, (w - image_size[1]) // 2
    return image[y:y + image_size[0], x:x + image_size[1]]


def central_crop_v2(image: np.ndarray, center_crop_fraction: float = 0.875) -> np.ndarray:
    """Centre square whose side is ``fraction`` of the shorter edge."""
    h, w = image.shape[:2]
    side = int(round(center_crop_fraction * min(h, w)))
    y, x = (h - side + 1) // 2, (w - side + 1) // 2
    return image[y:y + side, x:x + side]


def crop_augment_whiten(image: np.ndarray, *, is_training: bool, image_size: Sequence[int],
                        eval_resize: Optional[Sequence[int]] = None, use_whitening: bool = True,
                        center_crop_fraction: float = 0.875, rng: Rng = None) -> np.ndarray:
    """Training: random crop, resize, random flip.  Evaluation: resize the shorter side to
    ``eval_resize`` (default ``image_size / fraction``) and take the centre window -- or the
    centre square of ``fraction`` resized, when ``eval_resize`` is None."""
    if is_training:
        rng = rng or np.random.default_rng()
        out = resize_bilinear(random_crop(image, rng=rng), image_size)
        if rng.uniform() > 0.5:
            out = out[:, ::-1]
    elif eval_resize is not None:
        out = central_crop(resize_bilinear(image, eval_resize), image_size)
    else:
        out = resize_bilinear(central_crop_v2(image, center_crop_fraction), image_size)
    out = np.ascontiguousarray(out, dtype=np.float32)
    return whiten(out) if use_whitening else out


def image_processor(*, is_training: bool, image_size: Sequence[int], num_classes: Optional[int] = None,
                    eval_resize: Optional[Sequence[int]] = None, use_whitening: bool = True, seed: int = 0,
                    channels_first: bool = True) -> Callable[[dict], dict]:
    """Per-example function: ``{"image", "label"}`` -> ``{"image" [C, H, W] float32, "label" int}``."""
    counter = {"n": 0}

    def fn(example: dict) -> dict:
        rng = np.random.default_rng((seed, example.get("_index", counter["n"])))
        counter["n"] += 1
        img = crop_augment_whiten(np.asarray(example["image"]), is_training=is_training, image_size=image_size,
                                  eval_resize=eval_resize, use_whitening=use_whitening, rng=rng)
        if channels_first:
            img = np.ascontiguousarray(img.transpose(2, 0, 1))
        label = np.int64(example["label"])
        if num_classes is not None and not 0 <= label < num_classes:
            raise ValueError(f"label {label} outside [0, {num_classes})")
        return {"image": img, "label": label}

    return fn


def pad_with_negative_labels(example: dict) -> dict:
    """The padding example of evaluation batches: zero image, label -1 (ignored by the metrics)."""
    return {"image": np.zeros_like(example["image"]), "label": np.int64(-1)}


class ImagenetInput(input_pipeline.PipelineInput):
    """``source`` yields ``{"image" [H, W, 3], "label"}``; this input applies the ImageNet train /
    eval recipe and batches (reference ``ImagenetInput``, :376-393)."""

    @config_class
    class Config(input_pipeline.PipelineInput.Config):
        image_size: Sequence[int] = (224, 224)
        eval_resize: Optional[Sequence[int]] = None
        num_classes: Optional[int] = 1000
        use_whitening: bool = True
        seed: int = 0

    def _make_source(self):
        cfg = self._config
        raw_source = super()._make_source()
        proc = image_processor(is_training=cfg.is_training, image_size=cfg.image_size, num_classes=cfg.num_classes,
                               eval_resize=cfg.eval_resize, use_whitening=cfg.use_whitening, seed=cfg.seed)
        return lambda index, count: raw_source(index, count).filter(is_valid_image).map(proc)


def is_valid_image(example: dict) -> bool:
    """Drops records whose image failed to decode (empty, or not ``[H, W, 3]``)."""
    img = np.asarray(example.get("image"))
    return img.ndim == 3 and img.shape[2] == 3 and img.shape[0] > 0 and img.shape[1] > 0


def fake_image_source(*, num_examples: int = 8, image_size: Sequence[int] = (40, 56), num_classes: int = 10,
                      seed: int = 0):
    """``source(shard_index, shard_count)`` of synthetic labelled images (reference
    ``fake_image_dataset``, :410-438)."""

    def make(index: int, count: int):
        rng = np.random.default_rng(seed)
        rows = [{"image": rng.integers(0, 256, (image_size[0], image_size[1], 3), dtype=np.uint8),
                 "label": int(rng.integers(0, num_classes)), "_index": i} for i in range(num_examples)]
        return input_pipeline.read(input_pipeline.ListSource(rows), shard_index=index, shard_count=count,
                                   num_epochs=None)

    return make
