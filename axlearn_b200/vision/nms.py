"""Batched, padded non-maximum suppression (reference: axlearn/vision/nms.py:119-230).

``non_max_suppression_padded(scores, boxes, max_output_size, iou_threshold)`` takes boxes SORTED by
decreasing score (padding boxes, of zero area, last) and returns exactly ``max_output_size`` scores
and boxes per image, zero-filled past the number kept -- static shapes, so that the heads after it
run with one set of kernels whatever the image holds.

The reference walks the boxes tile by tile inside a while loop.  Here the greedy result is computed
as the fixed point of a data-parallel rule over the whole ``[B, N, N]`` overlap matrix:

    keep[j] = not any(keep[i] and overlap[i, j] for i < j)

started from "keep everything".  Each sweep is one masked reduction; after sweep ``t`` the verdicts
of all boxes whose chain of suppressors is shorter than ``t`` are final, so the number of sweeps is
the longest such chain (a handful in practice), never more than ``N``, and the result equals the
sequential algorithm's exactly.
"""

from __future__ import annotations

import torch

from axlearn_b200.vision import similarity_ops

Tensor = torch.Tensor


def nms_keep_mask(boxes: Tensor, *, iou_threshold: float) -> Tensor:
    """``boxes`` ``[B, N, 4]`` in decreasing score order -> bool ``[B, N]``: survives greedy NMS.
    Zero-area boxes overlap nothing, so they survive; callers drop them by their padding."""
    n = boxes.shape[1]
    iou = similarity_ops.pairwise_iou(boxes_a=boxes, boxes_b=boxes)
    earlier = torch.ones(n, n, dtype=torch.bool, device=boxes.device).triu(diagonal=1)      # [i, j]: i < j
    over = (iou > iou_threshold) & earlier
    keep = torch.ones(boxes.shape[:2], dtype=torch.bool, device=boxes.device)
    for _ in range(n):
        new_keep = ~(over & keep[:, :, None]).any(dim=1)
        if torch.equal(new_keep, keep):
            break
        keep = new_keep
    return keep


def non_max_suppression_padded(scores: Tensor, boxes: Tensor, max_output_size: int,
                               iou_threshold: float) -> tuple[Tensor, Tensor]:
    """``scores`` ``[B, N]`` (decreasing), ``boxes`` ``[B, N, 4]`` -> ``([B, max_output_size],
    [B, max_output_size, 4])``: the kept boxes in score order, then zeros."""
    b, n = scores.shape
    valid = similarity_ops.areas(boxes) > 0
    keep = nms_keep_mask(boxes, iou_threshold=iou_threshold) & valid
    # Stable compaction: kept positions first, in their original order.
    order = torch.arange(n, device=scores.device).expand(b, n)
    idx = torch.where(keep, order, order + n).argsort(dim=-1)[:, :max_output_size]
    if idx.shape[1] < max_output_size:
        idx = torch.cat([idx, idx.new_zeros(b, max_output_size - idx.shape[1])], dim=1)
    count = keep.sum(dim=-1).clamp(max=max_output_size)
    live = torch.arange(max_output_size, device=scores.device)[None] < count[:, None]
    out_scores = torch.gather(scores, 1, idx) * live.to(scores.dtype)
    out_boxes = torch.gather(boxes, 1, idx[..., None].expand(-1, -1, 4)) * live[..., None].to(boxes.dtype)
    return out_scores, out_boxes


def multiclass_nms_padded(scores: Tensor, boxes: Tensor, *, max_output_size_per_class: int, max_total_size: int,
                          iou_threshold: float, score_threshold: float = 0.0) -> dict:
    """Per-class NMS then the best ``max_total_size`` detections of all classes.

    ``scores`` ``[B, N, C]``, ``boxes`` ``[B, N, 4]`` (shared by the classes) or ``[B, N, C, 4]``.
    Returns ``detection_boxes [B, T, 4]``, ``detection_scores [B, T]``, ``detection_classes [B, T]``
    (int) and ``num_detections [B]``; classes are processed as one batch of ``B * C`` problems."""
    b, n, c = scores.shape
    if boxes.ndim == 3:
        boxes = boxes[:, :, None, :].expand(b, n, c, 4)
    s = scores.permute(0, 2, 1).reshape(b * c, n)
    bx = boxes.permute(0, 2, 1, 3).reshape(b * c, n, 4)
    s = torch.where(s > score_threshold, s, torch.zeros_like(s))
    bx = bx * (s > 0)[..., None].to(bx.dtype)                    # below the threshold: a padding box
    s, order = s.sort(dim=-1, descending=True, stable=True)
    bx = torch.gather(bx, 1, order[..., None].expand(-1, -1, 4))
    k = min(max_output_size_per_class, n)
    ks, kb = non_max_suppression_padded(s, bx, k, iou_threshold)
    ks, kb = ks.reshape(b, c * k), kb.reshape(b, c * k, 4)
    classes = torch.arange(c, device=scores.device).repeat_interleave(k)[None].expand(b, -1)
    t = min(max_total_size, c * k)
    top_s, top_i = ks.topk(t, dim=-1)
    out = {"detection_scores": top_s,
           "detection_boxes": torch.gather(kb, 1, top_i[..., None].expand(-1, -1, 4)),
           "detection_classes": torch.gather(classes, 1, top_i) * (top_s > 0).long(),
           "num_detections": (top_s > 0).sum(dim=-1)}
    if t < max_total_size:
        pad = max_total_size - t
        out["detection_scores"] = torch.nn.functional.pad(out["detection_scores"], (0, pad))
        out["detection_boxes"] = torch.nn.functional.pad(out["detection_boxes"], (0, 0, 0, pad))
        out["detection_classes"] = torch.nn.functional.pad(out["detection_classes"], (0, pad))
    return out
