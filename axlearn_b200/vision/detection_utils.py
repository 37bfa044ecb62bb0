"""Box utilities for object detection (all boxes ``[..., 4]`` as ``(ymin, xmin, ymax, xmax)``).

Parity targets in the reference: axlearn/vision/utils_detection.py (IoU / box coding / clipping),
axlearn/vision/anchor.py (``AnchorGenerator``: per pyramid level, ``scales`` x ``aspect_ratios``
anchors of base size ``anchor_size * 2^level`` centred on every stride cell),
axlearn/vision/nms.py (score-sorted greedy non-maximum suppression with padding to a fixed
count) and axlearn/vision/roi_aligner.py (bilinear ROI align).
"""

from __future__ import annotations

from typing import Sequence

import torch

Tensor = torch.Tensor


def box_area(boxes: Tensor) -> Tensor:
    return (boxes[..., 2] - boxes[..., 0]).clamp_min(0) * (boxes[..., 3] - boxes[..., 1]).clamp_min(0)


def pairwise_iou(a: Tensor, b: Tensor) -> Tensor:
    """``a [N, 4]``, ``b [M, 4]`` -> ``[N, M]``."""
    top_left = torch.maximum(a[:, None, :2], b[None, :, :2])
    bottom_right = torch.minimum(a[:, None, 2:], b[None, :, 2:])
    inter = (bottom_right - top_left).clamp_min(0).prod(dim=-1)
    union = box_area(a)[:, None] + box_area(b)[None] - inter
    return torch.where(union > 0, inter / union.clamp_min(1e-12), torch.zeros_like(inter))


def clip_boxes(boxes: Tensor, image_shape: Sequence[int]) -> Tensor:
    h, w = image_shape
    hi = torch.tensor([h, w, h, w], dtype=boxes.dtype, device=boxes.device)
    return torch.minimum(boxes.clamp_min(0), hi)


def encode_boxes(boxes: Tensor, anchors: Tensor, weights: Sequence[float] = (1.0, 1.0, 1.0, 1.0)) -> Tensor:
    """Faster-RCNN box coding ``(dy, dx, dh, dw)`` of ``boxes`` relative to ``anchors``."""
    ah, aw = anchors[..., 2] - anchors[..., 0], anchors[..., 3] - anchors[..., 1]
    ay, ax = anchors[..., 0] + 0.5 * ah, anchors[..., 1] + 0.5 * aw
    bh, bw = boxes[..., 2] - boxes[..., 0], boxes[..., 3] - boxes[..., 1]
    by, bx = boxes[..., 0] + 0.5 * bh, boxes[..., 1] + 0.5 * bw
    wy, wx, wh, ww = weights
    return torch.stack([wy * (by - ay) / ah, wx * (bx - ax) / aw,
                        wh * torch.log(bh / ah), ww * torch.log(bw / aw)], dim=-1)


def decode_boxes(deltas: Tensor, anchors: Tensor, weights: Sequence[float] = (1.0, 1.0, 1.0, 1.0)) -> Tensor:
    ah, aw = anchors[..., 2] - anchors[..., 0], anchors[..., 3] - anchors[..., 1]
    ay, ax = anchors[..., 0] + 0.5 * ah, anchors[..., 1] + 0.5 * aw
    wy, wx, wh, ww = weights
    cy, cx = deltas[..., 0] / wy * ah + ay, deltas[..., 1] / wx * aw + ax
    h = torch.exp((deltas[..., 2] / wh).clamp(max=4.135)) * ah
    w = torch.exp((deltas[..., 3] / ww).clamp(max=4.135)) * aw
    return torch.stack([cy - 0.5 * h, cx - 0.5 * w, cy + 0.5 * h, cx + 0.5 * w], dim=-1)


def generate_anchors(*, image_shape: Sequence[int], min_level: int, max_level: int, num_scales: int = 3,
                     aspect_ratios: Sequence[float] = (1.0, 2.0, 0.5), anchor_size: float = 4.0) -> dict:
    """``{level: [H_l * W_l * A, 4]}``: at every cell centre of stride ``2^level``, anchors of area
    ``(anchor_size * 2^level * 2^(s / num_scales))^2`` and the given height / width ratios."""
    out = {}
    for level in range(min_level, max_level + 1):
        stride = 2 ** level
        hs = torch.arange(stride / 2, image_shape[0], stride)
        ws = torch.arange(stride / 2, image_shape[1], stride)
        cy, cx = torch.meshgrid(hs, ws, indexing="ij")
        shapes = []
        for s in range(num_scales):
            base = anchor_size * stride * 2 ** (s / num_scales)
            for ratio in aspect_ratios:
                shapes.append((base * ratio ** 0.5, base / ratio ** 0.5))       # (height, width)
        hw = torch.tensor(shapes)
        centers = torch.stack([cy, cx], dim=-1).reshape(-1, 1, 2)
        half = hw.reshape(1, -1, 2) / 2
        out[level] = torch.cat([centers - half, centers + half], dim=-1).reshape(-1, 4)
    return out


def non_max_suppression(boxes: Tensor, scores: Tensor, *, iou_threshold: float = 0.5, max_output_size: int = 100,
                        score_threshold: float = float("-inf")):
    """Greedy NMS.  Returns ``(indices [max_output_size], valid [max_output_size])`` with indices
    padded by -1 (fixed-size output, as the reference's jit-friendly form)."""
    order = torch.argsort(scores, descending=True, stable=True)
    order = order[scores[order] > score_threshold]
    iou = pairwise_iou(boxes[order], boxes[order])
    keep = []
    suppressed = torch.zeros(len(order), dtype=torch.bool)
    for i in range(len(order)):
        if suppressed[i]:
            continue
        keep.append(int(order[i]))
        if len(keep) == max_output_size:
            break
        suppressed |= iou[i] > iou_threshold
    idx = torch.full((max_output_size,), -1, dtype=torch.long)
    idx[:len(keep)] = torch.tensor(keep, dtype=torch.long)
    return idx, idx >= 0


def roi_align(features: Tensor, boxes: Tensor, *, output_size: int = 7, sampling_ratio: int = 2) -> Tensor:
    """``features [H, W, C]`` (one image, one level; coordinates in feature-map units), ``boxes
    [N, 4]`` -> ``[N, output_size, output_size, C]``: every output cell averages ``sampling_ratio^2``
    bilinear samples."""
    h, w, c = features.shape
    n = boxes.shape[0]
    s = output_size * sampling_ratio
    frac = (torch.arange(s, dtype=torch.float32, device=features.device) + 0.5) / s
    ys = boxes[:, 0:1] + frac[None] * (boxes[:, 2:3] - boxes[:, 0:1])          # [N, s]
    xs = boxes[:, 1:2] + frac[None] * (boxes[:, 3:4] - boxes[:, 1:2])
    # Sample positions are pixel centres: shift by half a pixel, clamp to the map.
    ys, xs = (ys - 0.5).clamp(0, h - 1), (xs - 0.5).clamp(0, w - 1)
    y0, x0 = ys.floor().long(), xs.floor().long()
    y1, x1 = (y0 + 1).clamp(max=h - 1), (x0 + 1).clamp(max=w - 1)
    wy, wx = (ys - y0.float())[:, :, None, None], (xs - x0.float())[:, None, :, None]
    f = features.float()

    def at(yy, xx):
        return f[yy[:, :, None], xx[:, None, :]]                               # [N, s, s, C]

    top = at(y0, x0) * (1 - wx) + at(y0, x1) * wx
    bottom = at(y1, x0) * (1 - wx) + at(y1, x1) * wx
    samples = top * (1 - wy) + bottom * wy
    return samples.reshape(n, output_size, sampling_ratio, output_size, sampling_ratio, c).mean(dim=(2, 4)).to(features.dtype)
