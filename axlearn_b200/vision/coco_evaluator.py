"""COCO-style detection metrics: AP averaged over IoU 0.50:0.95, AP50, AP75, size buckets, AR.

Covers the role of axlearn/vision/coco_evaluator.py and eval_detection.py, which hand detections to
pycocotools; that package is not a dependency here, so the protocol is implemented directly:
per image and class, detections in score order are matched greedily to the unmatched ground truth
of highest IoU above the threshold (crowd / ignored boxes absorb matches without counting);
precision is made monotone and sampled at 101 recall points.
"""

from __future__ import annotations

from collections import defaultdict
from typing import Optional, Sequence

import numpy as np

IOU_THRESHOLDS = np.linspace(0.5, 0.95, 10)
RECALL_POINTS = np.linspace(0.0, 1.0, 101)
AREA_RANGES = {"all": (0, 1e10), "small": (0, 32 ** 2), "medium": (32 ** 2, 96 ** 2), "large": (96 ** 2, 1e10)}


def _iou(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``[N, 4] x [M, 4] -> [N, M]`` for ``(y0, x0, y1, x1)`` boxes."""
    if a.size == 0 or b.size == 0:
        return np.zeros((len(a), len(b)))
    tl = np.maximum(a[:, None, :2], b[None, :, :2])
    br = np.minimum(a[:, None, 2:], b[None, :, 2:])
    inter = np.prod(np.clip(br - tl, 0, None), axis=-1)
    area = lambda x: np.prod(np.clip(x[:, 2:] - x[:, :2], 0, None), axis=-1)
    return inter / np.maximum(area(a)[:, None] + area(b)[None] - inter, 1e-12)


class COCOEvaluator:
    def __init__(self, max_detections: Sequence[int] = (1, 10, 100)):
        self._max_dets = tuple(max_detections)
        self.reset()

    def reset(self) -> None:
        self._gt = defaultdict(list)       # (image, class) -> [(box, ignore)]
        self._dt = defaultdict(list)       # (image, class) -> [(box, score)]
        self._classes: set = set()

    def add_groundtruth(self, image_id, boxes, classes, is_crowd: Optional[Sequence] = None) -> None:
        for i, (box, c) in enumerate(zip(np.asarray(boxes, dtype=np.float64), np.asarray(classes))):
            if int(c) < 0:
                continue
            self._gt[(image_id, int(c))].append((box, bool(is_crowd[i]) if is_crowd is not None else False))
            self._classes.add(int(c))

    def add_detections(self, image_id, boxes, scores, classes) -> None:
        for box, s, c in zip(np.asarray(boxes, dtype=np.float64), np.asarray(scores), np.asarray(classes)):
            self._dt[(image_id, int(c))].append((box, float(s)))
            self._classes.add(int(c))

    def _match(self, key, area_range, max_det):
        """Per IoU threshold: for every detection (score order) matched / ignored flags."""
        gts = self._gt.get(key, [])
        dts = sorted(self._dt.get(key, []), key=lambda d: -d[1])[:max_det]
        g_boxes = np.array([g[0] for g in gts]).reshape(-1, 4)
        g_area = np.prod(g_boxes[:, 2:] - g_boxes[:, :2], axis=-1) if len(gts) else np.zeros(0)
        g_ignore = np.array([g[1] for g in gts], dtype=bool) | (g_area < area_range[0]) | (g_area > area_range[1])
        order = np.argsort(g_ignore, kind="stable")                  # counted ground truth first
        g_boxes, g_ignore = g_boxes[order], g_ignore[order]
        crowd = np.array([g[1] for g in gts], dtype=bool)[order] if len(gts) else np.zeros(0, dtype=bool)
        d_boxes = np.array([d[0] for d in dts]).reshape(-1, 4)
        d_scores = np.array([d[1] for d in dts])
        iou = _iou(d_boxes, g_boxes)
        t_n = len(IOU_THRESHOLDS)
        d_match = np.zeros((t_n, len(dts)), dtype=bool)
        d_ignore = np.zeros((t_n, len(dts)), dtype=bool)
        for ti, thr in enumerate(IOU_THRESHOLDS):
            taken = np.zeros(len(gts), dtype=bool)
            for di in range(len(dts)):
                best, best_g = min(thr, 1 - 1e-10), -1
                for gi in range(len(gts)):
                    if taken[gi] and not crowd[gi]:
                        continue
                    if best_g > -1 and not g_ignore[best_g] and g_ignore[gi]:
                        break                                        # a counted match beats ignored ones
                    if iou[di, gi] < best:
                        continue
                    best, best_g = iou[di, gi], gi
                if best_g > -1:
                    taken[best_g] = True
                    d_match[ti, di] = True
                    d_ignore[ti, di] = g_ignore[best_g]
        d_area = np.prod(d_boxes[:, 2:] - d_boxes[:, :2], axis=-1) if len(dts) else np.zeros(0)
        outside = (d_area < area_range[0]) | (d_area > area_range[1])
        d_ignore |= (~d_match) & outside[None]
        return d_scores, d_match, d_ignore, int((~g_ignore).sum())

    def _accumulate(self, area: str, max_det: int):
        """precision ``[T, R, K]`` and recall ``[T, K]`` (-1 where a class has no ground truth)."""
        classes = sorted(self._classes)
        images = sorted({k[0] for k in list(self._gt) + list(self._dt)}, key=str)
        precision = -np.ones((len(IOU_THRESHOLDS), len(RECALL_POINTS), len(classes)))
        recall = -np.ones((len(IOU_THRESHOLDS), len(classes)))
        for ki, c in enumerate(classes):
            scores, matches, ignores, num_gt = [], [], [], 0
            for img in images:
                s, m, ig, n = self._match((img, c), AREA_RANGES[area], max_det)
                scores.append(s), matches.append(m), ignores.append(ig)
                num_gt += n
            if num_gt == 0:
                continue
            s = np.concatenate(scores)
            order = np.argsort(-s, kind="mergesort")
            m = np.concatenate(matches, axis=1)[:, order]
            ig = np.concatenate(ignores, axis=1)[:, order]
            tp = np.cumsum(m & ~ig, axis=1).astype(np.float64)
            fp = np.cumsum(~m & ~ig, axis=1).astype(np.float64)
            for ti in range(len(IOU_THRESHOLDS)):
                rc = tp[ti] / num_gt
                pr = tp[ti] / np.maximum(tp[ti] + fp[ti], np.spacing(1))
                recall[ti, ki] = rc[-1] if len(rc) else 0.0
                for i in range(len(pr) - 1, 0, -1):
                    pr[i - 1] = max(pr[i - 1], pr[i])
                idx = np.searchsorted(rc, RECALL_POINTS, side="left")
                q = np.zeros(len(RECALL_POINTS))
                ok = idx < len(pr)
                q[ok] = pr[idx[ok]]
                precision[ti, :, ki] = q
        return precision, recall

    def evaluate(self) -> dict:
        def mean(x):
            x = x[x > -1]
            return float(x.mean()) if x.size else -1.0

        big = self._max_dets[-1]
        p_all, r_all = self._accumulate("all", big)
        out = {"AP": mean(p_all), "AP50": mean(p_all[0]), "AP75": mean(p_all[5])}
        for area, tag in (("small", "APs"), ("medium", "APm"), ("large", "APl")):
            p, r = self._accumulate(area, big)
            out[tag] = mean(p)
            out["AR" + tag[2]] = mean(r)
        for m in self._max_dets:
            _, r = self._accumulate("all", m)
            out[f"ARmax{m}"] = mean(r)
        return out
