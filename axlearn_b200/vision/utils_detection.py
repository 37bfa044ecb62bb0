"""Box utilities for detection models and their inputs (reference:
axlearn/vision/utils_detection.py:27-1121).  Boxes are ``[..., 4]`` tensors, ``[ymin, xmin, ymax,
xmax]`` unless a ``BoxFormat`` says otherwise; everything broadcasts over leading dimensions."""

from __future__ import annotations

import enum
import functools
import math
from typing import Callable, Optional, Sequence, Union

import torch

Tensor = torch.Tensor


def _check_boxes(boxes: Tensor) -> None:
    if boxes.shape[-1] != 4:
        raise ValueError(f"boxes.shape[-1] is {boxes.shape[-1]}, but must be 4.")


def _hwhw(image_shape: Union[Tensor, Sequence[int]], like: Tensor) -> Tensor:
    """``[..., 2]`` (height, width) -> ``[..., 4]`` (height, width, height, width)."""
    shape = torch.as_tensor(image_shape, dtype=like.dtype, device=like.device)
    return torch.cat([shape, shape], dim=-1)


def normalize_boxes(*, boxes: Tensor, image_shape: Union[Tensor, Sequence[int]]) -> Tensor:
    """Pixel coordinates -> fractions of the image.  ``image_shape``: ``[2]`` or broadcastable ``[..., 1, 2]``."""
    _check_boxes(boxes)
    return boxes / _hwhw(image_shape, boxes)


def denormalize_boxes(*, boxes: Tensor, image_shape: Union[Tensor, Sequence[int]]) -> Tensor:
    _check_boxes(boxes)
    return boxes * _hwhw(image_shape, boxes)


def clip_boxes(boxes: Tensor, image_shape: Union[Tensor, Sequence[int]]) -> Tensor:
    """Clips to ``[0, height] x [0, width]``."""
    _check_boxes(boxes)
    return torch.minimum(boxes, _hwhw(image_shape, boxes)).clamp(min=0.0)


def sorted_top_k(values: Tensor, *, k: int) -> Tensor:
    """Indices of the ``k`` largest entries of the last axis, largest first; among equal values the
    LATER index comes first (the order of a reversed ascending sort)."""
    return values.argsort(dim=-1, stable=True).flip(-1)[..., :k]


def resize_and_crop_boxes(boxes: Tensor, image_scale: Tensor, output_size: Sequence[int], offset: Tensor) -> Tensor:
    """Boxes of an image that was scaled by ``image_scale`` (y, x) and then cropped at ``offset``
    (y0, x0) to ``output_size``."""
    scale = torch.as_tensor(image_scale, dtype=boxes.dtype, device=boxes.device)
    off = torch.as_tensor(offset, dtype=boxes.dtype, device=boxes.device)
    return clip_boxes(boxes * torch.cat([scale, scale], dim=-1) - torch.cat([off, off], dim=-1), output_size)


def get_non_empty_box_indices(boxes: Tensor) -> Tensor:
    """Indices (first axis) of ``[N, 4]`` boxes with positive height and width."""
    return ((boxes[:, 2] - boxes[:, 0] > 0) & (boxes[:, 3] - boxes[:, 1] > 0)).nonzero().flatten()


def compute_padded_size(desired_size: Sequence[int], stride: int) -> list:
    """The smallest (height, width) >= ``desired_size`` whose sides are multiples of ``stride``."""
    return [int(math.ceil(d / stride) * stride) for d in desired_size]


def process_source_id(source_id: Union[str, bytes, int]) -> int:
    """A numeric id from a string one ("" -> -1), as COCO-style evaluators want."""
    if isinstance(source_id, bytes):
        source_id = source_id.decode("utf-8")
    if isinstance(source_id, str):
        return int(source_id) if source_id.strip() else -1
    return int(source_id)


def multi_level_flatten(multi_level_inputs: dict, last_dim: Optional[int] = None) -> Tensor:
    """``{level: [B, ...]}`` -> ``[B, total]`` or ``[B, total, last_dim]``, levels in dict order."""
    parts = []
    for value in multi_level_inputs.values():
        b = value.shape[0]
        parts.append(value.reshape(b, -1, last_dim) if last_dim is not None else value.reshape(b, -1))
    return torch.cat(parts, dim=1)


def clip_or_pad_to_fixed_size(input_tensor: Tensor, size: int, constant_values: float = 0) -> Tensor:
    """First axis cut or padded (with ``constant_values``) to ``size``."""
    t = input_tensor[:size]
    if t.shape[0] == size:
        return t
    pad = torch.full((size - t.shape[0], *t.shape[1:]), constant_values, dtype=t.dtype, device=t.device)
    return torch.cat([t, pad], dim=0)


def pad_groundtruths_to_fixed_size(groundtruths: dict, size: int) -> dict:
    """Pads the box annotations (``boxes``, ``areas``, ``classes`` with -1, ``is_crowds`` with 0)."""
    out = dict(groundtruths)
    for key, fill in (("boxes", -1), ("is_crowds", 0), ("areas", -1), ("classes", -1)):
        out[key] = clip_or_pad_to_fixed_size(groundtruths[key], size, fill)
    return out


def filter_boxes_by_scores(boxes: Tensor, scores: Tensor, min_score_threshold: float) -> tuple[Tensor, Tensor]:
    """Boxes scoring at most the threshold become zeros and their scores -1 (shapes unchanged)."""
    _check_boxes(boxes)
    keep = scores > min_score_threshold
    return boxes * keep[..., None].to(boxes.dtype), torch.where(keep, scores, -torch.ones_like(scores))


def yxyx_to_xywh(boxes):
    """``[ymin, xmin, ymax, xmax] -> [xmin, ymin, width, height]`` (COCO's annotation format)."""
    _check_boxes(boxes)
    stack = torch.stack if isinstance(boxes, Tensor) else __import__("numpy").stack
    return stack([boxes[..., 1], boxes[..., 0], boxes[..., 3] - boxes[..., 1], boxes[..., 2] - boxes[..., 0]], -1)


class BoxFormat(str, enum.Enum):
    YminXminYmaxXmax = "YminXminYmaxXmax"      # the detectors' format
    XminYminXmaxYmax = "XminYminXmaxYmax"
    YminXminHW = "YminXminHW"
    XminYminWH = "XminYminWH"
    CxCyWH = "CxCyWH"


def _to_yxyx(b: Tensor, fmt: BoxFormat) -> Tensor:
    a0, a1, a2, a3 = b.unbind(-1)
    if fmt == BoxFormat.YminXminYmaxXmax:
        return b
    if fmt == BoxFormat.XminYminXmaxYmax:
        return torch.stack([a1, a0, a3, a2], -1)
    if fmt == BoxFormat.YminXminHW:
        return torch.stack([a0, a1, a0 + a2, a1 + a3], -1)
    if fmt == BoxFormat.XminYminWH:
        return torch.stack([a1, a0, a1 + a3, a0 + a2], -1)
    if fmt == BoxFormat.CxCyWH:
        return torch.stack([a1 - 0.5 * a3, a0 - 0.5 * a2, a1 + 0.5 * a3, a0 + 0.5 * a2], -1)
    raise NotImplementedError(fmt)


def _from_yxyx(b: Tensor, fmt: BoxFormat) -> Tensor:
    ymin, xmin, ymax, xmax = b.unbind(-1)
    if fmt == BoxFormat.YminXminYmaxXmax:
        return b
    if fmt == BoxFormat.XminYminXmaxYmax:
        return torch.stack([xmin, ymin, xmax, ymax], -1)
    if fmt == BoxFormat.YminXminHW:
        return torch.stack([ymin, xmin, ymax - ymin, xmax - xmin], -1)
    if fmt == BoxFormat.XminYminWH:
        return torch.stack([xmin, ymin, xmax - xmin, ymax - ymin], -1)
    if fmt == BoxFormat.CxCyWH:
        return torch.stack([0.5 * (xmin + xmax), 0.5 * (ymin + ymax), xmax - xmin, ymax - ymin], -1)
    raise NotImplementedError(fmt)


def transform_boxes(boxes: Tensor, source_format: BoxFormat, target_format: BoxFormat) -> Tensor:
    """Any of the five formats to any other (through the corner form)."""
    _check_boxes(boxes)
    if source_format == target_format:
        return boxes
    return _from_yxyx(_to_yxyx(boxes, BoxFormat(source_format)), BoxFormat(target_format))


def reshape_box_decorator(func: Callable) -> Callable:
    """Lets a function written for ``[N, 4]`` boxes take ``[..., 4]``: leading dimensions are
    flattened for the call and restored on a tensor result whose first dimension is ``N``."""

    @functools.wraps(func)
    def wrapper(boxes: Tensor, *args, **kwargs):
        lead = boxes.shape[:-1]
        out = func(boxes.reshape(-1, 4), *args, **kwargs)
        if isinstance(out, Tensor) and out.shape[:1] == (math.prod(lead),):
            return out.reshape(*lead, *out.shape[1:])
        return out

    return wrapper
