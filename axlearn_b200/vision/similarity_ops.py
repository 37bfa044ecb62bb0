"""Box similarity measures (reference: axlearn/vision/similarity_ops.py:12-181).

Boxes are ``[..., 4]`` in corner form ``[ymin, xmin, ymax, xmax]``.  Pairwise functions compare every
box of ``boxes_a`` (``[..., N, 4]``) with every box of ``boxes_b`` (``[..., M, 4]``); element-wise ones
compare boxes at the same position.  Comparisons that involve a padding box yield ``fill_value``.
"""

from __future__ import annotations

from typing import Optional

import torch

Tensor = torch.Tensor


def areas(boxes: Tensor) -> Tensor:
    return (boxes[..., 2] - boxes[..., 0]) * (boxes[..., 3] - boxes[..., 1])


def pairwise_intersection_areas(*, boxes_a: Tensor, boxes_b: Tensor) -> Tensor:
    a, b = boxes_a[..., :, None, :], boxes_b[..., None, :, :]
    heights = (torch.minimum(a[..., 2], b[..., 2]) - torch.maximum(a[..., 0], b[..., 0])).clamp(min=0.0)
    widths = (torch.minimum(a[..., 3], b[..., 3]) - torch.maximum(a[..., 1], b[..., 1])).clamp(min=0.0)
    return heights * widths


def _fill(values: Tensor, fill_loc: Tensor, fill_value: float) -> Tensor:
    return torch.where(fill_loc, torch.full_like(values, fill_value), values)


def _pair_paddings(boxes_a, boxes_b, paddings_a, paddings_b) -> Tensor:
    if paddings_a is None:
        paddings_a = torch.zeros(boxes_a.shape[:-1], dtype=torch.bool, device=boxes_a.device)
    if paddings_b is None:
        paddings_b = torch.zeros(boxes_b.shape[:-1], dtype=torch.bool, device=boxes_b.device)
    return paddings_a[..., :, None] | paddings_b[..., None, :]


def _safe_ratio(num: Tensor, den: Tensor) -> Tensor:
    """``num / den`` where ``num > 0``, else 0 (no division by an empty union or area)."""
    positive = num > 0.0
    return torch.where(positive, num / torch.where(positive, den, torch.ones_like(den)), torch.zeros_like(num))


def pairwise_iou(*, boxes_a: Tensor, boxes_b: Tensor, paddings_a: Optional[Tensor] = None,
                 paddings_b: Optional[Tensor] = None, fill_value: float = -1.0) -> Tensor:
    """``[..., N, M]`` intersection over union."""
    inter = pairwise_intersection_areas(boxes_a=boxes_a, boxes_b=boxes_b)
    unions = areas(boxes_a)[..., :, None] + areas(boxes_b)[..., None, :] - inter
    return _fill(_safe_ratio(inter, unions), _pair_paddings(boxes_a, boxes_b, paddings_a, paddings_b), fill_value)


def pairwise_ioa(*, boxes_a: Tensor, boxes_b: Tensor, paddings_a: Optional[Tensor] = None,
                 paddings_b: Optional[Tensor] = None, fill_value: float = -1.0) -> Tensor:
    """``[..., N, M]`` intersection over the area of the box of ``boxes_a`` (e.g. how much of a
    candidate lies inside a crowd region)."""
    inter = pairwise_intersection_areas(boxes_a=boxes_a, boxes_b=boxes_b)
    area_a = areas(boxes_a)[..., :, None].expand_as(inter)
    return _fill(_safe_ratio(inter, area_a), _pair_paddings(boxes_a, boxes_b, paddings_a, paddings_b), fill_value)


def elementwise_intersection_areas(*, boxes_a: Tensor, boxes_b: Tensor) -> Tensor:
    heights = (torch.minimum(boxes_a[..., 2], boxes_b[..., 2]) - torch.maximum(boxes_a[..., 0], boxes_b[..., 0])).clamp(min=0.0)
    widths = (torch.minimum(boxes_a[..., 3], boxes_b[..., 3]) - torch.maximum(boxes_a[..., 1], boxes_b[..., 1])).clamp(min=0.0)
    return heights * widths


def elementwise_iou(*, boxes_a: Tensor, boxes_b: Tensor, paddings_a: Optional[Tensor] = None,
                    paddings_b: Optional[Tensor] = None, fill_value: float = -1.0) -> Tensor:
    """``[..., N]`` IoU of boxes at equal positions."""
    inter = elementwise_intersection_areas(boxes_a=boxes_a, boxes_b=boxes_b)
    unions = areas(boxes_a) + areas(boxes_b) - inter
    fill_loc = torch.zeros(inter.shape, dtype=torch.bool, device=inter.device)
    if paddings_a is not None:
        fill_loc = fill_loc | paddings_a
    if paddings_b is not None:
        fill_loc = fill_loc | paddings_b
    return _fill(_safe_ratio(inter, unions), fill_loc, fill_value)
