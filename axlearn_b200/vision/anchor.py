"""Multi-level anchors and their labelling with ground truth (reference:
axlearn/vision/anchor.py:25-282)."""

from __future__ import annotations

import dataclasses
import itertools
from typing import Optional, Sequence

import numpy as np
import torch

from axlearn_b200.vision import matchers

Tensor = torch.Tensor


@dataclasses.dataclass
class AnchorLabels:
    """Ground truth matched to anchors.  ``groundtruth_boxes`` ``[B, N, 4]`` (zeros unless the
    match is foreground); ``groundtruth_classes`` ``[B, N, ...]`` (-1 unless foreground);
    ``box_paddings`` ``[B, N]`` True for every non-foreground match; ``class_paddings`` True for
    ignored matches only (background anchors do train the classifier); ``anchor_boxes`` ``[N, 4]``."""

    groundtruth_boxes: Tensor
    groundtruth_classes: Tensor
    box_paddings: Tensor
    class_paddings: Tensor
    anchor_boxes: Tensor


class AnchorLabeler:
    """Labels a batch of images against one shared set of anchors.  Matched boxes are returned as
    they are (encoding them relative to the anchors is the loss's business)."""

    def __init__(self, box_matcher_cfg: Optional[matchers.Matcher.Config] = None):
        self.box_matcher = (box_matcher_cfg or matchers.ArgmaxMatcher.default_config()).instantiate()

    def __call__(self, *, per_level_anchor_boxes: dict, groundtruth_boxes: Tensor,
                 groundtruth_classes: Tensor) -> AnchorLabels:
        results = self.box_matcher.match(per_level_anchor_boxes, groundtruth_boxes)
        foreground = results.labels == matchers.FOREGROUND
        background = results.labels == matchers.BACKGROUND
        index = results.matches.reshape(results.matches.shape + (1,) * (groundtruth_classes.ndim - 2))
        classes = torch.gather(groundtruth_classes, 1, index.expand(*results.matches.shape, *groundtruth_classes.shape[2:]))
        fg_c = foreground.reshape(index.shape)
        classes = torch.where(fg_c, classes, torch.full_like(classes, -1))
        boxes = torch.gather(groundtruth_boxes, 1, results.matches[..., None].expand(-1, -1, 4))
        boxes = torch.where(foreground[..., None], boxes, torch.zeros_like(boxes))
        return AnchorLabels(groundtruth_boxes=boxes, groundtruth_classes=classes, box_paddings=~foreground,
                            class_paddings=~(foreground | background), anchor_boxes=results.anchor_boxes[0])


class AnchorGenerator:
    """Anchors of ``num_scales`` octave-fractions x ``aspect_ratios`` (width / height) at every cell
    centre of levels ``min_level .. max_level``; an anchor of level ``l`` has area
    ``(anchor_size * 2^l * 2^(s / num_scales))^2``."""

    def __init__(self, *, min_level: int = 3, max_level: int = 7, num_scales: int = 3,
                 aspect_ratios: Sequence[float] = (0.5, 1.0, 2.0), anchor_size: float = 4.0):
        self.min_level, self.max_level, self.num_scales = min_level, max_level, num_scales
        self.aspect_ratios, self.anchor_size = tuple(aspect_ratios), anchor_size

    def __call__(self, image_size: Sequence[int]) -> dict:
        """``{str(level): [H_l * W_l * num_scales * len(aspect_ratios), 4]}``; within a level, cells
        in row-major order, and within a cell scale-major, aspect-minor."""
        out = {}
        for level in range(self.min_level, self.max_level + 1):
            stride = 2 ** level
            y = np.arange(stride / 2, image_size[0], stride)
            x = np.arange(stride / 2, image_size[1], stride)
            xv, yv = np.meshgrid(x, y)
            xv, yv = xv.reshape(-1).astype(np.float32), yv.reshape(-1).astype(np.float32)
            per_shape = []
            for scale, aspect in itertools.product(range(self.num_scales), self.aspect_ratios):
                base = self.anchor_size * stride * 2 ** (scale / float(self.num_scales))
                half_x, half_y = base * aspect ** 0.5 / 2.0, base * aspect ** -0.5 / 2.0
                per_shape.append(np.stack([yv - half_y, xv - half_x, yv + half_y, xv + half_x], axis=-1))
            out[str(level)] = torch.from_numpy(np.stack(per_shape, axis=-2).reshape(-1, 4).astype(np.float32))
        return out
