"""Matchers that pair anchors with ground-truth boxes (reference: axlearn/vision/matchers.py:19-420).

Every anchor gets exactly one ground-truth index (``matches``) and a label saying what kind of
match it is (``labels``: FOREGROUND / BACKGROUND / IGNORE); a ground-truth box may be matched by any
number of anchors.  Padding boxes (all coordinates negative) never match.  Everything is batched
tensor arithmetic -- no loop over images or boxes -- so it runs on the device where the boxes are.
"""

from __future__ import annotations

import dataclasses
import enum

import torch

from axlearn_b200.common.config import Configurable, config_class
from axlearn_b200.vision import similarity_ops

Tensor = torch.Tensor

FOREGROUND = 1
IGNORE = -2
BACKGROUND = -1


@dataclasses.dataclass
class MatchResults:
    """``matches`` int ``[B, N]`` in ``[0, M)``; ``labels`` int32 ``[B, N]``; ``anchor_boxes`` float
    ``[1 or B, N, 4]``: the per-level anchors concatenated."""

    matches: Tensor
    labels: Tensor
    anchor_boxes: Tensor


class Matcher(Configurable):
    @config_class
    class Config(Configurable.Config):
        # Match types, for increasing similarity.
        labels: list = [BACKGROUND, IGNORE, FOREGROUND]

    def match(self, per_level_anchor_boxes: dict, groundtruth_boxes: Tensor) -> MatchResults:
        """``per_level_anchor_boxes``: ``{level: [num_anchors, 4]}`` (shared by the batch);
        ``groundtruth_boxes``: ``[B, M, 4]``."""
        raise NotImplementedError(type(self))


def _expand_anchor_dims(*, anchor_boxes: Tensor, groundtruth_boxes: Tensor) -> Tensor:
    if anchor_boxes.ndim == groundtruth_boxes.ndim:
        return anchor_boxes
    if anchor_boxes.ndim == groundtruth_boxes.ndim - 1:
        return anchor_boxes[None]
    raise ValueError(f"Expected anchor boxes dimension is 2 or 3 but got {anchor_boxes.ndim}")


def _similarity(per_level_anchor_boxes: dict, groundtruth_boxes: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    anchors = torch.cat(list(per_level_anchor_boxes.values()), dim=0).to(groundtruth_boxes.device)
    anchors = _expand_anchor_dims(anchor_boxes=anchors, groundtruth_boxes=groundtruth_boxes)
    gt_padding = groundtruth_boxes.amax(dim=-1) < 0.0
    sim = similarity_ops.pairwise_iou(boxes_a=anchors, boxes_b=groundtruth_boxes, paddings_a=anchors.amax(dim=-1) < 0.0,
                                      paddings_b=gt_padding, fill_value=-1.0)
    return anchors, gt_padding, sim          # sim: [B, N, M]


class ArgmaxMatcher(Matcher):
    """Each anchor takes its most similar ground-truth box; ``thresholds`` (ascending) cut the
    similarity into ``len(labels)`` strata.  With ``force_match_columns`` the best anchor of every
    ground-truth box is made FOREGROUND for that box even when its similarity is below the cut."""

    @config_class
    class Config(Matcher.Config):
        thresholds: list = [0.5, 0.5]
        force_match_columns: bool = True

    def __init__(self, cfg):
        super().__init__(cfg)
        cfg = self._config
        if len(cfg.labels) != len(cfg.thresholds) + 1:
            raise ValueError(f"len(labels) must be len(thresholds) + 1, got {len(cfg.labels)} and {len(cfg.thresholds)}")
        if sorted(cfg.thresholds) != list(cfg.thresholds):
            raise ValueError("`thresholds` must be sorted.")
        self.labels = list(cfg.labels)
        self.thresholds = [-float("inf")] + list(cfg.thresholds) + [float("inf")]

    def match(self, per_level_anchor_boxes: dict, groundtruth_boxes: Tensor) -> MatchResults:
        anchors, _, sim = _similarity(per_level_anchor_boxes, groundtruth_boxes)
        match_vals, matches = sim.max(dim=-1)
        labels = torch.zeros_like(matches, dtype=torch.int32)
        for label, low, high in zip(self.labels, self.thresholds[:-1], self.thresholds[1:]):
            labels = torch.where((match_vals >= low) & (match_vals < high), torch.full_like(labels, label), labels)
        if self._config.force_match_columns:
            num_rows = sim.shape[-2]
            best_rows = sim.argmax(dim=1)                                       # [B, M]
            # A row may be the best of several columns: the lowest column index wins, as an argmax
            # over the one-hot [B, M, N] matrix would give.
            cols = torch.arange(sim.shape[-1], device=sim.device).expand_as(best_rows)
            forced_col = torch.full((sim.shape[0], num_rows), sim.shape[-1], dtype=torch.long, device=sim.device)
            forced_col.scatter_reduce_(1, best_rows, cols, reduce="amin", include_self=True)
            forced = forced_col < sim.shape[-1]
            matches = torch.where(forced, forced_col, matches)
            labels = torch.where(forced, torch.full_like(labels, self.labels[-1]), labels)
        return MatchResults(matches=matches, labels=labels, anchor_boxes=anchors)


class DistanceType(enum.Enum):
    L2 = 1
    IOU = 2


class ATSSMatcher(Matcher):
    """Adaptive Training Sample Selection (arXiv:1912.02424): per ground-truth box take the ``top_k``
    closest anchors of every pyramid level as candidates, set the IoU threshold of the box to the
    mean plus the standard deviation of its candidates' IoUs, and make FOREGROUND the candidates
    over the threshold whose centre lies inside the box the anchor is matched to."""

    @config_class
    class Config(Matcher.Config):
        top_k: int = 9
        distance_type: DistanceType = DistanceType.IOU

    def __init__(self, cfg):
        super().__init__(cfg)
        self.labels = list(self._config.labels)

    @staticmethod
    def _centers(boxes: Tensor) -> tuple[Tensor, Tensor]:
        return (boxes[..., 0] + boxes[..., 2]) / 2, (boxes[..., 1] + boxes[..., 3]) / 2

    def match(self, per_level_anchor_boxes: dict, groundtruth_boxes: Tensor) -> MatchResults:
        cfg = self._config
        anchors, gt_padding, sim = _similarity(per_level_anchor_boxes, groundtruth_boxes)
        matches = sim.argmax(dim=-1)                                            # [B, N]
        matched_gt = torch.gather(groundtruth_boxes, 1, matches[..., None].expand(-1, -1, 4))
        labels = torch.full_like(matches, self.labels[0], dtype=torch.int32)
        gt_cy, gt_cx = self._centers(groundtruth_boxes)                         # [B, M]
        sim_t = sim.transpose(1, 2)                                             # [B, M, N]
        cand_idx, cand_iou, start = [], [], 0
        for level_boxes in per_level_anchor_boxes.values():
            n = level_boxes.shape[0]
            if cfg.distance_type == DistanceType.L2:
                a_cy, a_cx = self._centers(level_boxes.to(groundtruth_boxes.device))
                dist = -torch.sqrt((a_cx[None, None, :] - gt_cx[..., None]) ** 2 + (a_cy[None, None, :] - gt_cy[..., None]) ** 2)
            elif cfg.distance_type == DistanceType.IOU:
                dist = sim_t[..., start:start + n]
            else:
                raise NotImplementedError(f"ATSS matcher distance type {cfg.distance_type} is not implemented.")
            top = dist.topk(min(cfg.top_k, n), dim=-1).indices + start
            cand_idx.append(top)
            cand_iou.append(torch.gather(sim_t, -1, top))
            start += n
        cand_idx, cand_iou = torch.cat(cand_idx, dim=-1), torch.cat(cand_iou, dim=-1)   # [B, M, C]
        thresholds = cand_iou.mean(dim=-1) + cand_iou.std(dim=-1, unbiased=False)
        positive = (cand_iou >= thresholds[..., None]) & ~gt_padding[..., None]
        # Anchors that are a positive candidate of some box.
        num_anchors = matches.shape[1]
        hit = torch.zeros(matches.shape[0], num_anchors + 1, dtype=torch.bool, device=matches.device)
        flat = torch.where(positive, cand_idx, torch.full_like(cand_idx, num_anchors)).reshape(matches.shape[0], -1)
        hit.scatter_(1, flat, torch.ones_like(flat, dtype=torch.bool))
        a_cy, a_cx = self._centers(anchors)
        inside = ((a_cy > matched_gt[..., 0]) & (a_cy < matched_gt[..., 2])
                  & (a_cx > matched_gt[..., 1]) & (a_cx < matched_gt[..., 3]))
        labels = torch.where(hit[:, :num_anchors] & inside, torch.full_like(labels, self.labels[-1]), labels)
        return MatchResults(matches=matches, labels=labels, anchor_boxes=anchors)
